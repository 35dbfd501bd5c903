// Fused wave epilogue shared by the tensor-core kernels: bias, activation, residual order rule, FP16
// rounding and the coalesced row stores.
#pragma once
#include "k44_kernels.cuh"

namespace k44b {

// ---------------------------------------------------------------------------------------------------
// fused epilogue (semantics of kernels/cuda/kernel44_cuda_pack.cuh:54-58, 69-126; GELU added)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
    case 1: return fmaxf(v, 0.0f);
    case 2: return 1.0f / (1.0f + __expf(-v));
    case 3: return v / (1.0f + __expf(-v));
    case 4: return fmaxf(v, 0.1f * v);
    case 5: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    default: return v;
    }
}

// residual goes in before the activation when an output-row map is present, after it otherwise
__device__ __forceinline__ float finish_value(float acc, float bias, float res, int act, bool has_res, bool has_map) {
    float v = acc + bias;
    if (has_res && has_map) v += res;
    v = apply_act(v, act);
    if (has_res && !has_map) v += res;
    return v;
}

__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// ---- peer exchange of neuron-sharded plans (see PeerArgs) ------------------------------------------------------
// 16-byte piece of an output row -> the same element offset of every peer canvas
__device__ __forceinline__ void store_to_peers(const PeerArgs *p, uint64_t elem_off, const uint4 &val) {
    const uint32_t n = p->n_peers;
    for (uint32_t q = 0; q < n; ++q) *reinterpret_cast<uint4 *>(p->canvas[q] + elem_off) = val;
}
// One thread per CTA, after the CTA's last store and a CTA barrier that all storing threads passed: one system-scope
// fence covers the CTA's stores to the peers (fences are cumulative over what the barrier ordered before them); the
// CTA that arrives last closes the launch and publishes the new launch count to every peer.
__device__ __forceinline__ void peer_signal_done(const PeerArgs *p, uint32_t ctas_in_launch) {
    __threadfence_system();
    const uint32_t prev = atomicAdd(p->sync + kSyncDone, 1u);
    if (prev + 1u == ctas_in_launch) {
        __threadfence();
        p->sync[kSyncDone] = 0u;
        const uint32_t epoch = p->sync[kSyncEpoch] + 1u;
        p->sync[kSyncEpoch] = epoch;
        // one system-scope fence orders everything this launch stored (the other CTAs' stores through their own fences and
        // the counter) before the count words below; the words themselves can then be plain system-scope stores that go out
        // back to back instead of each waiting for the one before it
        __threadfence_system();
        const uint32_t n = p->n_peers;
        for (uint32_t q = 0; q < n; ++q) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p->arrive[q]), "r"(epoch) : "memory");
    }
}
// One thread, before the launch reads the canvas: every peer must have finished the launches this one depends on — all but
// the last `slack` of the launches this rank has completed itself (slack 0: every earlier launch; the host raises it for
// launches that neither read what the peers' latest launches write nor overwrite what they read).
// Bounded: returns false when a peer does not show up within `limit` cycles.
__device__ __forceinline__ bool peer_wait_ready(const PeerArgs *p, unsigned long long limit, uint32_t slack) {
    const uint32_t need = *reinterpret_cast<volatile uint32_t *>(p->sync + kSyncEpoch) - slack;
    const uint32_t n = p->n_peers;
    const long long t0 = clock64();
    for (;;) {
        bool all = true;
        for (uint32_t q = 0; q < n; ++q) {
            uint32_t v;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p->sync + q) : "memory");
            all = all && (int32_t)(v - need) >= 0;
        }
        if (all) break;
        if ((unsigned long long)(clock64() - t0) > limit) return false;
    }
    __threadfence_system();        // acquire side: the peers' rows stored before their count words are visible from here on
    return true;
}

// Branch-free activation for the tensor-core epilogue: the activation kind is a template parameter so that the
// 32 values a thread converts are independent straight-line code (a per-element runtime switch serialises them
// behind branch latency when only one warp runs per scheduler).
// GELU(v) = v * Phi(v) with Phi(v) = 1 / (1 + exp(-v * P(v^2))): the logit of the normal distribution function is
// odd and smooth, and a quadratic P in v^2, fitted on |v| <= 9 (beyond it Phi is 0 or 1 to 1e-11 and v is clamped
// for the exponent only), reproduces the erf form of GELU to 2.6e-5 absolute — forty times below the FP16 rounding
// of the stored result at |v| = 2. Two special-function instructions and eight FP32 operations per value, no
// branch. (libm's erff costs several times as much and made the epilogue of GELU waves the bottleneck of the
// tensor-core kernels.) The coefficients carry the factor -log2(e) of the base-2 exponential.
// A variant with one special-function instruction per value — sigmoid, SiLU and this GELU through tanh.approx — stayed inside
// the output tolerance for every FP16 pre-activation, but it is ten times less accurate (up to 2.5e-4 * |v|) and bought under
// 1 % on the power-capped token-shift benchmark; it was dropped.
__device__ __forceinline__ float gelu_fast(float v) {
    const float vc = fminf(fmaxf(v, -9.0f), 9.0f);
    const float v2 = vc * vc;
    float p = fmaf(v2, 0.0010164447594434023f, -0.10678916424512863f);
    p = fmaf(v2, p, -2.3011064529418945f);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(vc * p));       // exp(-v P(v^2))
    return __fdividef(v, 1.0f + e);
}

template <int ACT>
__device__ __forceinline__ float act_fast(float v) {
    if (ACT == 1) return fmaxf(v, 0.0f);
    if (ACT == 2) return __fdividef(1.0f, 1.0f + __expf(-v));
    if (ACT == 3) return __fdividef(v, 1.0f + __expf(-v));
    if (ACT == 4) return fmaxf(v, 0.1f * v);
    if (ACT == 5) return gelu_fast(v);
    return v;
}

// Each thread converts its 32 values (one neuron, 32 columns) to FP16 and parks them in a padded shared-memory
// slot; the warp then writes the 32 rows back as whole 64-byte pieces (8 rows per instruction), so that every
// global store fills complete 32-byte sectors. Must be called by all 32 lanes of a warp.
template <int ACT, bool RES, bool MAP>
__device__ __forceinline__ void stage_and_store_t(const WaveArgs &a, const float (&v)[32], float bias, bool live, uint32_t oj,
                                                  uint64_t col0, uint8_t *wstage, uint32_t lane) {
    uint4 *slot = reinterpret_cast<uint4 *>(wstage + lane * 80u);
    uint32_t pk[16];
    if (RES) {
        const uint4 *rsrc = reinterpret_cast<const uint4 *>(a.canvas + a.res_off + (uint64_t)oj * a.pitch + col0);
        uint4 rv[4];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) rv[q4] = live ? rsrc[q4] : make_uint4(0, 0, 0, 0);
        const __half2 *rh = reinterpret_cast<const __half2 *>(rv);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float2 r = __half22float2(rh[e]);
            float lo = v[2 * e] + bias, hi = v[2 * e + 1] + bias;
            if (MAP) { lo += r.x; hi += r.y; }
            lo = act_fast<ACT>(lo); hi = act_fast<ACT>(hi);
            if (!MAP) { lo += r.x; hi += r.y; }
            const __half2 h2 = __floats2half2_rn(lo, hi);
            pk[e] = *reinterpret_cast<const uint32_t *>(&h2);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const __half2 h2 = __floats2half2_rn(act_fast<ACT>(v[2 * e] + bias), act_fast<ACT>(v[2 * e + 1] + bias));
            pk[e] = *reinterpret_cast<const uint32_t *>(&h2);
        }
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) slot[q4] = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
    __syncwarp();
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t r = 8u * i + (lane >> 2), piece = lane & 3u;
        const uint32_t oj_r = __shfl_sync(0xffffffffu, oj, r);
        const int live_r = __shfl_sync(0xffffffffu, live ? 1 : 0, r);
        const uint4 val = *reinterpret_cast<const uint4 *>(wstage + r * 80u + piece * 16u);
        if (live_r) {
            const uint64_t off = a.y_off + (uint64_t)oj_r * a.pitch + col0 + piece * 8u;
            *reinterpret_cast<uint4 *>(a.canvas + off) = val;
            if (a.peers) store_to_peers(a.peers, off, val);
        }
    }
    __syncwarp();
}

// ---- tile store through shared memory and tensor copies --------------------------------------------------------
// The 128 epilogue threads build a 128-row x 64-column block of the output tile in shared memory (rows of 128 bytes, the
// 16-byte chunk c of row r at chunk position c ^ (r & 7): the 128-byte swizzle, so that the eight rows a quarter-warp
// writes at once fall into distinct banks) and one thread hands the block to the copy engine: one tensor copy into this
// rank's canvas and, in a neuron-sharded plan, one per peer canvas (WaveArgs::out_maps). The tensor maps describe exactly
// the wave's output rows ([cout][pitch] from y_off), so rows of a partial last tile are clipped by the copy itself.
// This function converts the 32 values (one neuron, 32 columns = half a block) a thread holds and parks them in the block.
template <int ACT, bool RES>
__device__ __forceinline__ void stage_half_block_t(const WaveArgs &a, const float (&v)[32], float bias, bool live, uint32_t j,
                                                   uint64_t col0, uint32_t block_smem, uint32_t r, uint32_t half) {
    uint32_t pk[16];
    if (RES) {
        const uint4 *rsrc = reinterpret_cast<const uint4 *>(a.canvas + a.res_off + (uint64_t)j * a.pitch + col0);
        uint4 rv[4];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) rv[q4] = live ? rsrc[q4] : make_uint4(0, 0, 0, 0);
        const __half2 *rh = reinterpret_cast<const __half2 *>(rv);
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float2 rr = __half22float2(rh[e]);
            const __half2 h2 = __floats2half2_rn(act_fast<ACT>(v[2 * e] + bias) + rr.x, act_fast<ACT>(v[2 * e + 1] + bias) + rr.y);
            pk[e] = *reinterpret_cast<const uint32_t *>(&h2);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const __half2 h2 = __floats2half2_rn(act_fast<ACT>(v[2 * e] + bias), act_fast<ACT>(v[2 * e + 1] + bias));
            pk[e] = *reinterpret_cast<const uint32_t *>(&h2);
        }
    }
    const uint32_t row_addr = block_smem + r * 128u;
#pragma unroll
    for (uint32_t q4 = 0; q4 < 4u; ++q4)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((half * 4u + q4) ^ (r & 7u)) << 4)), "r"(pk[4 * q4]),
                     "r"(pk[4 * q4 + 1]), "r"(pk[4 * q4 + 2]), "r"(pk[4 * q4 + 3])
                     : "memory");
}

// (no output-row map on this path: the residual is added after the activation)
__device__ __forceinline__ void stage_half_block(const WaveArgs &a, const float (&v)[32], float bias, bool live, uint32_t j, uint64_t col0,
                                                 uint32_t block_smem, uint32_t r, uint32_t half) {
#define K44B_STAGE_CASE(ACT)                                                                                      \
    if (a.has_residual) stage_half_block_t<ACT, true>(a, v, bias, live, j, col0, block_smem, r, half);            \
    else stage_half_block_t<ACT, false>(a, v, bias, live, j, col0, block_smem, r, half);                          \
    break;
    switch (a.act) {
    case 1: K44B_STAGE_CASE(1)
    case 2: K44B_STAGE_CASE(2)
    case 3: K44B_STAGE_CASE(3)
    case 4: K44B_STAGE_CASE(4)
    case 5: K44B_STAGE_CASE(5)
    default: K44B_STAGE_CASE(0)
    }
#undef K44B_STAGE_CASE
}

template <int ACT>
__device__ __forceinline__ void stage_and_store_a(const WaveArgs &a, const float (&v)[32], float bias, bool has_map, bool live, uint32_t oj,
                                                  uint64_t col0, uint8_t *wstage, uint32_t lane) {
    if (!a.has_residual) stage_and_store_t<ACT, false, false>(a, v, bias, live, oj, col0, wstage, lane);
    else if (has_map) stage_and_store_t<ACT, true, true>(a, v, bias, live, oj, col0, wstage, lane);
    else stage_and_store_t<ACT, true, false>(a, v, bias, live, oj, col0, wstage, lane);
}

// One uniform branch per 32 values instead of one per value.
__device__ __forceinline__ void stage_and_store(const WaveArgs &a, const float (&v)[32], float bias, bool has_map, bool live, uint32_t oj,
                                                uint64_t col0, uint8_t *wstage, uint32_t lane) {
    switch (a.act) {
    case 1: stage_and_store_a<1>(a, v, bias, has_map, live, oj, col0, wstage, lane); break;
    case 2: stage_and_store_a<2>(a, v, bias, has_map, live, oj, col0, wstage, lane); break;
    case 3: stage_and_store_a<3>(a, v, bias, has_map, live, oj, col0, wstage, lane); break;
    case 4: stage_and_store_a<4>(a, v, bias, has_map, live, oj, col0, wstage, lane); break;
    case 5: stage_and_store_a<5>(a, v, bias, has_map, live, oj, col0, wstage, lane); break;
    default: stage_and_store_a<0>(a, v, bias, has_map, live, oj, col0, wstage, lane); break;
    }
}

}  // namespace k44b
