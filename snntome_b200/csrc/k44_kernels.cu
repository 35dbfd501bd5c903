// Wave kernels for sm_100a.
//
//  * k44_wave_umma_kernel — the hot path: persistent, warp-specialised streaming kernel (template in
//    k44_stream_kernel.cuh, instantiated per tile width in k44_stream_n*.cu; dispatched from here).
//  * k44_wave_umma_cluster_kernel — small waves (fewer tiles than SMs): the K splits of a tile form a thread-block
//    cluster and reduce through distributed shared memory; written for programmatic dependent launch and for
//    grouped launches of independent waves.
//  * k44_wave_fma_kernel — general FP32-FMA path (any gather table, any element alignment, any group
//    size); also the cross-check for the tensor-core path.
//  * packer / conversion kernels.
//  (Token-shifted runs: k44_shift_kernel.cu. Element-wise and attention steps: k44_valu.cu. Epilogue and the peer
//  exchange of neuron-sharded plans: k44_epilogue.cuh.)
//
// Every wait on a barrier is bounded in time; on expiry the kernel records a status bit, drains its
// own copies, frees its tensor memory and returns.
#include "k44_kernels.cuh"
#include "k44_epilogue.cuh"
#include "k44_ptx.cuh"

namespace k44b {


// ---------------------------------------------------------------------------------------------------
// FMA path
// ---------------------------------------------------------------------------------------------------
// CTA = 256 threads = 16 neurons x one 64-column tile. Per 64-synapse stage the 64 gathered rows
// (2-byte loads: offsets may have any alignment — this is what lets a tap be a token shift) and the
// 16x64 weight block are staged in shared memory; thread (q, c) accumulates neurons 4q..4q+3 for
// column c.
constexpr int kFmaRows = 16;

__global__ void __launch_bounds__(256) k44_wave_fma_kernel(const WaveArgs a) {
    __shared__ __half xs[kStageK][64];
    __shared__ __align__(16) __half ws[kFmaRows][kStageK];
    __shared__ uint64_t offs[kStageK];
    __shared__ uint32_t shs[kStageK];

    const uint32_t tile = blockIdx.x % a.num_col_tiles64;                 // 64-column tile (one-dimensional grid: y stops at 65535 blocks)
    const uint32_t j0 = (blockIdx.x / a.num_col_tiles64) * kFmaRows;      // first neuron
    const uint32_t g = j0 / a.group;
    const uint32_t tid = threadIdx.x, c = tid & 63u, q = tid >> 6;
    const uint64_t tile_x = a.tile_off_x ? a.tile_off_x[tile] : (uint64_t)tile * 64u;       // where this tile's gathers are anchored
    const __half *xbase = a.canvas + a.x_base_off + tile_x;
    const uint64_t x_limit = a.canvas_elems - a.x_base_off - tile_x;   // exclusive bound for off + 64
    const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
    const uint32_t col_in_frame = (tile * 64u + c) % flen;

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    bool bad = false;
    for (uint32_t ks = 0; ks < a.num_kstages; ++ks) {
        if (tid < kStageK) {
            const uint32_t s = ks * kStageK + tid;
            uint64_t off = 0;
            uint32_t sh = 0;
            if (s < a.fan_in) {
                if (a.gather_mode == GATHER_IDX) {
                    off = a.gather[(uint64_t)g * a.fan_in + s];
                    if (a.shifts) sh = a.shifts[(uint64_t)g * a.fan_in + s];
                } else {
                    const uint32_t e = a.gather[(uint64_t)g * a.boxes_per_group + s / a.box_h];
                    off = (uint64_t)((e & kBoxRowMask) + s % a.box_h) * a.pitch;
                    sh = e >> 28;
                }
            }
            if (off + 64u > x_limit) { off = 0; bad = true; }   // record and skip instead of faulting
            offs[tid] = off;
            shs[tid] = sh;
        } else if (tid < kStageK + 128) {
            const uint32_t v = tid - kStageK, r = v >> 3, k8 = v & 7u;   // 16 rows x 8 vectors
            const uint4 wv = a.w_tiles[tiled_vec_index(j0 + r, ks * 8u + k8, a.num_kstages)];
            *reinterpret_cast<uint4 *>(&ws[r][k8 * 8]) = wv;
        }
        __syncthreads();
        if (a.has_shift) {
#pragma unroll 4
            for (uint32_t k = q; k < kStageK; k += 4) {
                const uint32_t sh = shs[k];
                xs[k][c] = col_in_frame >= sh ? xbase[offs[k] + c - sh] : __float2half(0.0f);
            }
        } else {
#pragma unroll 4
            for (uint32_t k = q; k < kStageK; k += 4) xs[k][c] = xbase[offs[k] + c];
        }
        __syncthreads();
#pragma unroll 8
        for (uint32_t k = 0; k < kStageK; ++k) {
            const float x = __half2float(xs[k][c]);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = fmaf(__half2float(ws[q * 4 + i][k]), x, acc[i]);
        }
        __syncthreads();
    }
    if (bad) atomicOr(a.status, (uint32_t)ST_BAD_INDEX);
    uint64_t tile_y = (uint64_t)tile * 64u;
    if (a.tile_off_y) {
        const uint32_t e = a.tile_off_y[tile];
        tile_y = a.tile_mask ? (uint64_t)(e & 0xffffu) << 2 : e;
        if (a.tile_mask && !((e >> (16u + (c >> 2))) & 1u)) return;        // this column's quad is halo, not pixels
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t j = j0 + q * 4 + i;
        if (j >= a.cout) continue;
        const uint32_t oj = a.cout_map ? a.cout_map[j] : j;
        const uint64_t o = (uint64_t)oj * a.pitch + tile_y + c;
        const float b = a.bias ? __half2float(a.bias[j]) : 0.0f;
        const float r = a.has_residual ? __half2float(a.canvas[a.res_off + o]) : 0.0f;
        a.canvas[a.y_off + o] = __float2half_rn(finish_value(acc[i], b, r, a.act, a.has_residual != 0, a.cout_map != nullptr));
    }
}

cudaError_t launch_wave_fma(const WaveArgs &a, cudaStream_t s) {
    const uint64_t blocks = (uint64_t)a.num_col_tiles64 * ((a.cout + kFmaRows - 1) / kFmaRows);
    if (blocks == 0 || blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    dim3 grid((uint32_t)blocks);
    k44_wave_fma_kernel<<<grid, 256, 0, s>>>(a);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------
// tcgen05 path
// ---------------------------------------------------------------------------------------------------
constexpr int kUmmaThreads = 192;

cudaError_t launch_wave_umma(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s) {
    if (a.k_splits == 0 || a.kstages_per_split == 0) return cudaErrorInvalidValue;
    if (a.k_splits > 1 && (!a.scratch || !a.counters)) return cudaErrorInvalidValue;
    if (a.box_h != 1u && a.box_h < 8u) return cudaErrorInvalidValue;
    switch (d.n_tile) {          // one translation unit per tile width (k44_stream_n*.cu)
    case 64: return launch_wave_umma_n64(a, d, tmap, num_sms, s);
    case 128: return launch_wave_umma_n128(a, d, tmap, num_sms, s);
    case 256: return launch_wave_umma_n256(a, d, tmap, num_sms, s);
    default: return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------------------------------------------
// tcgen05 path for small waves: one work item per CTA, K splits of a tile form a thread-block cluster
// ---------------------------------------------------------------------------------------------------
// A wave with fewer 128-neuron tiles than SMs (every linear of a decoder at decode batch sizes) cuts each
// tile's fan-in into S = 1, 2, 4 or 8 splits. The S CTAs of a tile are launched as one cluster and combine
// their FP32 partial accumulators through distributed shared memory: CTA r owns rows [r*128/S, (r+1)*128/S) of
// the tile, every CTA writes the partial sums of those rows into the owner's receive buffer, one cluster
// barrier later each owner adds its S partials, applies the epilogue and stores its rows. No global scratch,
// no atomics, bit-reproducible. The kernel is also written for programmatic dependent launch: barrier set-up,
// tensor-memory allocation and the weight copies of the first stages are issued before it waits for the
// previous wave, because weights never depend on it.
namespace smallwave {
constexpr uint32_t kXBytes = kStageK * 128u;                         // one 64-column block
constexpr uint32_t kStageBytes = kStageWBytes + kXBytes;             // 24 KiB
constexpr uint32_t kRecvBytes = 36864u;                              // [src rank][group of 4 columns][owned rows + 1 pad][4 floats], largest for 16 splits
constexpr uint32_t smem_bytes(int stages) { return 1024u + (uint32_t)stages * kStageBytes + kRecvBytes + 256u; }
constexpr uint32_t kTmemCols = 64u;
// 3 stages: two CTAs per SM (waves with up to 2 x SMs work items); 7 stages: one CTA per SM with a deep pipeline

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float x, float y, float z, float w) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Owner side of the exchange, compile-time split count: thread t of the 128 epilogue threads sums the S partial
// rows for 64/S columns of one owned row, applies the epilogue and stores 16-byte pieces.
template <int S, int ACT>
__device__ __forceinline__ void finish_owned_t(const WaveArgs &a, const float *recv, uint32_t t, uint32_t mt, uint32_t ct, uint32_t rank) {
    constexpr uint32_t rows_owned = kTileM / S, ncol = 64u / S;
    const uint32_t row_local = t / S, col0 = (t % S) * ncol;
    const uint32_t j = mt * kTileM + rank * rows_owned + row_local;
    float v[ncol];
#pragma unroll
    for (uint32_t c = 0; c < ncol; c += 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (uint32_t src = 0; src < (uint32_t)S; ++src) {
            const float4 p = *reinterpret_cast<const float4 *>(recv + (((size_t)src * 16u + (col0 + c) / 4u) * (rows_owned + 1u) + row_local) * 4u);
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        v[c] = acc.x; v[c + 1] = acc.y; v[c + 2] = acc.z; v[c + 3] = acc.w;
    }
    if (j >= a.cout) return;
    const bool has_map = a.cout_map != nullptr;
    const uint32_t oj = has_map ? a.cout_map[j] : j;
    const float bias = a.bias ? __half2float(a.bias[j]) : 0.0f;
    const uint64_t o = (uint64_t)oj * a.pitch + (uint64_t)ct * 64u + col0;
    __half *dst = a.canvas + a.y_off + o;
    if constexpr (ncol == 4u) {  // 16 splits: four values (8 bytes) per thread
        float r[4] = {0.f, 0.f, 0.f, 0.f};
        if (a.has_residual) {
            const uint2 rv = *reinterpret_cast<const uint2 *>(a.canvas + a.res_off + o);
            const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
            const float2 f0 = __half22float2(rh[0]), f1 = __half22float2(rh[1]);
            r[0] = f0.x; r[1] = f0.y; r[2] = f1.x; r[3] = f1.y;
        }
        uint32_t pk[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float lo = v[2 * e] + bias, hi = v[2 * e + 1] + bias;
            if (has_map) { lo += r[2 * e]; hi += r[2 * e + 1]; }
            lo = act_fast<ACT>(lo); hi = act_fast<ACT>(hi);
            if (!has_map) { lo += r[2 * e]; hi += r[2 * e + 1]; }
            const __half2 h2 = __floats2half2_rn(lo, hi);
            pk[e] = *reinterpret_cast<const uint32_t *>(&h2);
        }
        *reinterpret_cast<uint2 *>(dst) = make_uint2(pk[0], pk[1]);
        if (a.peers) {
            const uint32_t n = a.peers->n_peers;
            for (uint32_t q = 0; q < n; ++q) *reinterpret_cast<uint2 *>(a.peers->canvas[q] + a.y_off + o) = make_uint2(pk[0], pk[1]);
        }
    } else {
#pragma unroll
    for (uint32_t c = 0; c + 8u <= ncol; c += 8) {
        float r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (a.has_residual) {
            const uint4 rv = *reinterpret_cast<const uint4 *>(a.canvas + a.res_off + o + c);
            const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(rh[e]); r[2 * e] = f.x; r[2 * e + 1] = f.y; }
        }
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float lo = v[c + 2 * e] + bias, hi = v[c + 2 * e + 1] + bias;
            if (has_map) { lo += r[2 * e]; hi += r[2 * e + 1]; }
            lo = act_fast<ACT>(lo); hi = act_fast<ACT>(hi);
            if (!has_map) { lo += r[2 * e]; hi += r[2 * e + 1]; }
            const __half2 h2 = __floats2half2_rn(lo, hi);
            pk[e] = *reinterpret_cast<const uint32_t *>(&h2);
        }
        const uint4 val = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        *reinterpret_cast<uint4 *>(dst + c) = val;
        if (a.peers) store_to_peers(a.peers, a.y_off + o + c, val);
    }
    }
}

template <int S>
__device__ __forceinline__ void finish_owned(const WaveArgs &a, const float *recv, uint32_t t, uint32_t mt, uint32_t ct, uint32_t rank) {
    switch (a.act) {
    case 1: finish_owned_t<S, 1>(a, recv, t, mt, ct, rank); break;
    case 2: finish_owned_t<S, 2>(a, recv, t, mt, ct, rank); break;
    case 3: finish_owned_t<S, 3>(a, recv, t, mt, ct, rank); break;
    case 4: finish_owned_t<S, 4>(a, recv, t, mt, ct, rank); break;
    case 5: finish_owned_t<S, 5>(a, recv, t, mt, ct, rank); break;
    default: finish_owned_t<S, 0>(a, recv, t, mt, ct, rank); break;
    }
}
}  // namespace smallwave

template <int kStages>
__global__ void __launch_bounds__(kUmmaThreads, kStages <= 3 ? 2 : 1)
k44_wave_umma_cluster_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ WaveGroupArgs grp, const UmmaDesc d) {
    using namespace smallwave;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_smem = smem_base;
    const uint32_t x_smem = smem_base + kStages * kStageWBytes;
    const uint32_t recv_smem = x_smem + kStages * kXBytes;
    const uint32_t ctl = recv_smem + kRecvBytes;
    const uint32_t full_bar = ctl, empty_bar = ctl + 8u * kStages, tfull_bar = ctl + 16u * kStages;
    uint8_t *base_ptr = smem_raw + (smem_base - ptx::smem_addr(smem_raw));
    float *recv = reinterpret_cast<float *>(base_ptr + kStages * kStageBytes);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + kStages * kStageBytes + kRecvBytes + 16 * kStages + 16);
    volatile uint32_t *abort_word = tmem_slot + 1;
    volatile uint32_t *epi_ok = tmem_slot + 2;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // which wave of the group this cluster belongs to (uniform per CTA)
    const uint32_t S = grp.splits;                         // == cluster size
    const uint32_t cid = blockIdx.x / S;
    uint32_t g = 0;
#pragma unroll
    for (uint32_t i = 1; i < (uint32_t)kMaxGroupWaves; ++i)
        if (i < grp.count && cid >= grp.first_cluster[i]) g = i;
    WaveArgs a = grp.w[0];
    if (g == 1) a = grp.w[1];
    else if (g == 2) a = grp.w[2];
    else if (g == 3) a = grp.w[3];
    const uint32_t tile = cid - grp.first_cluster[g], rank = cluster_rank();
    const uint32_t tiles_n = a.num_col_tiles64;
    const uint32_t mt = tile / tiles_n, ct = tile % tiles_n;
    const uint32_t ks0 = rank * a.kstages_per_split;
    const uint32_t ks1 = min(a.num_kstages, ks0 + a.kstages_per_split);   // may be empty for the last ranks
    const uint32_t boxes_per_stage = kStageK / a.box_h;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(full_bar + 8u * s, 1);
            ptx::mbar_init(empty_bar + 8u * s, 1);
        }
        ptx::mbar_init(tfull_bar, 1);
        *abort_word = 0;
        ptx::fence_mbar_init();
        // weights of the first stages do not depend on the previous wave: start them before anything else
        const uint64_t pol_w0 = ptx::policy_evict_first();
        const uint4 *wsrc0 = a.w_tiles + (uint64_t)mt * a.num_kstages * (kStageWBytes / 16u);
        const uint32_t nst0 = ks1 > ks0 ? ks1 - ks0 : 0u;
        for (uint32_t i = 0; i < (nst0 < (uint32_t)kStages ? nst0 : (uint32_t)kStages); ++i) {
            ptx::mbar_arrive_expect_tx(full_bar + 8u * i, kStageBytes);
            ptx::bulk_g2s(w_smem + i * kStageWBytes, wsrc0 + (uint64_t)(ks0 + i) * (kStageWBytes / 16u), kStageWBytes, full_bar + 8u * i, pol_w0);
        }
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (S > 1) cluster_arrive();            // phase A: "this CTA is alive"; waited for before the first remote write
    grid_launch_dependents();               // the next wave may start its own set-up and weight prefetch

    auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
        if (ptx::mbar_try_wait(bar, parity)) return true;      // the common case costs one instruction
        const long long t0 = clock64();
        for (uint32_t it = 0;; ++it) {
            if (ptx::mbar_try_wait(bar, parity)) return true;
            if ((it & 31u) == 31u) {
                if (*abort_word != 0u) return false;
                if ((unsigned long long)(clock64() - t0) > d.wait_cycles) return false;
            }
        }
    };

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) ptx::prefetch_tensormap(&tmap);
        const uint64_t pol_w = ptx::policy_evict_first();
        const uint64_t pol_x = ptx::policy_evict_last();
        const uint32_t *rows = a.gather + (uint64_t)(mt / a.mtiles_per_group) * a.boxes_per_group;
        const uint4 *wsrc = a.w_tiles + (uint64_t)mt * a.num_kstages * (kStageWBytes / 16u);
        const uint32_t nst = ks1 > ks0 ? ks1 - ks0 : 0u;
        const uint32_t pre = nst < (uint32_t)kStages ? nst : (uint32_t)kStages;
        // (the weights of the first `pre` stages were issued by thread 0 during set-up)
        // the run table is static too: fetch its first entries before waiting for the previous wave
        uint32_t cached_base = (ks0 * boxes_per_stage) & ~31u;
        uint32_t cached = (cached_base + lane < a.boxes_per_group) ? __ldg(rows + cached_base + lane) : 0u;
        grid_dependency_wait();             // everything below reads rows the previous wave wrote
        bool ok = true;
        if (a.peers) {                       // ... and, in a neuron-sharded plan, rows the peers stored into this canvas
            uint32_t okp = 1u;
            if (lane == 0) {
                okp = peer_wait_ready(a.peers, d.wait_cycles, a.peer_slack) ? 1u : 0u;
                if (!okp) { atomicOr(a.status, (uint32_t)ST_TIMEOUT_PEER); *abort_word = 1u; }
            }
            ok = __shfl_sync(0xffffffffu, okp, 0) != 0u;
        }
        fence_proxy_async_global();
        uint32_t issued = 0;
        for (uint32_t ks = ks0; ks < ks1 && ok; ++ks, ++issued) {
            const uint32_t stage = issued % kStages, ph = (issued / kStages) & 1u;
            if (issued >= pre) {
                if (lane == 0) {
                    ok = wait(empty_bar + 8u * stage, ph ^ 1u);
                    if (ok) {
                        ptx::mbar_arrive_expect_tx(full_bar + 8u * stage, kStageBytes);
                        ptx::bulk_g2s(w_smem + stage * kStageWBytes, wsrc + (uint64_t)ks * (kStageWBytes / 16u), kStageWBytes, full_bar + 8u * stage, pol_w);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
            }
            for (uint32_t b = 0; b < boxes_per_stage; ++b) {
                const uint32_t bi = ks * boxes_per_stage + b;
                if ((bi & ~31u) != cached_base) {
                    cached_base = bi & ~31u;
                    cached = (cached_base + lane < a.boxes_per_group) ? __ldg(rows + cached_base + lane) : 0u;
                }
                const uint32_t row = __shfl_sync(0xffffffffu, cached, bi & 31u) & kBoxRowMask;
                if (lane == 0)
                    ptx::tma_load_2d(x_smem + stage * kXBytes + b * a.box_h * 128u, &tmap, (int32_t)(ct * 64u), (int32_t)row, full_bar + 8u * stage, pol_x);
            }
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
            *abort_word = 1u;
            const uint32_t first = issued > (uint32_t)kStages ? issued - kStages : 0u;
            for (uint32_t i = first; i < issued; ++i) {
                const long long t0 = clock64();
                bool done = false;
                while (!done && (unsigned long long)(clock64() - t0) < d.wait_cycles)
                    done = ptx::mbar_try_wait(full_bar + 8u * (i % kStages), (i / kStages) & 1u);
                if (!done) atomicOr(a.status, (uint32_t)ST_TIMEOUT_DRAIN);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = true;
            uint32_t consumed = 0;
            for (uint32_t ks = ks0; ks < ks1; ++ks, ++consumed) {
                const uint32_t stage = consumed % kStages, ph = (consumed / kStages) & 1u;
                ok = wait(full_bar + 8u * stage, ph);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint64_t a0 = d.a_base | (uint64_t)(((w_smem + stage * kStageWBytes) >> 4) & 0x3fffu);
                const uint64_t b0 = d.b_base | (uint64_t)(((x_smem + stage * kXBytes) >> 4) & 0x3fffu);
#pragma unroll
                for (uint32_t k4 = 0; k4 < kStageK / 16u; ++k4)
                    ptx::umma_f16(tmem_base, a0 + (uint64_t)(k4 * d.a_k_step), b0 + (uint64_t)(k4 * d.b_k_step), d.idesc, (ks != ks0 || k4 != 0u) ? 1u : 0u);
                ptx::umma_commit(empty_bar + 8u * stage);
            }
            if (ok) ptx::umma_commit(tfull_bar);
            else { if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_MMA); *abort_word = 1u; }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: partial sums to their owners ----------------
        const uint32_t quarter = warp & 3u, r_in_tile = quarter * 32u + lane;
        const bool has_k = ks1 > ks0;
        if (threadIdx.x == 64u) epi_ok[0] = (!has_k || wait(tfull_bar, 0u)) ? 1u : 0u;
        epilogue_bar_sync();
        __syncwarp();
        grid_dependency_wait();             // already satisfied (the operands depended on it); orders this thread's own accesses
        const bool ok = epi_ok[0] != 0u;
        if (!ok && threadIdx.x == 64u) { if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_EPILOGUE); *abort_word = 1u; }
        ptx::tc_fence_after();
        const uint32_t rows_owned = kTileM / S;
        const uint32_t owner = r_in_tile / rows_owned, row_local = r_in_tile % rows_owned;
        // receive buffer of the owner: [src rank][group of 4 columns][row_local][4 floats] — the 16 or 32 lanes of a warp
        // that share an owner write one contiguous run per store instruction
        const uint32_t slot_off = (rank * 16u * (rows_owned + 1u) + row_local) * 16u;   // +1: padding row against bank conflicts on the read side
        if (S > 1) cluster_wait();          // phase A complete: every CTA of the cluster is running
        const uint32_t remote = S > 1 ? map_to_rank(recv_smem + slot_off, owner) : 0u;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < 64u; c0 += 32u) {
            uint32_t v[32];
            if (has_k && ok) {
                ptx::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + c0, v);
                ptx::tmem_ld_wait();
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = 0u;
            }
            if (S > 1) {
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                    st_cluster_v4(remote + ((c0 + e) / 4u) * (rows_owned + 1u) * 16u, __uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                                  __uint_as_float(v[e + 3]));
            } else {
#pragma unroll
                for (int e = 0; e < 32; e += 4)
                    *reinterpret_cast<float4 *>(recv + (((c0 + e) / 4u) * (rows_owned + 1u) + row_local) * 4u) =
                        make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
            }
        }
    }
    // ---------------- exchange complete -> every CTA finishes the rows it owns ----------------
    ptx::tc_fence_before();
    __syncwarp();
    if (S > 1) {
        if (warp < 2) cluster_wait();       // phase A (the epilogue warps waited for it above)
        cluster_arrive();                   // phase B: my partial sums are written
        cluster_wait();
    } else {
        __syncthreads();
    }
    if (warp >= 2 && *abort_word == 0u) {
        const uint32_t t = threadIdx.x - 64u;                       // 0..127
        switch (S) {
        case 1: finish_owned<1>(a, recv, t, mt, ct, rank); break;
        case 2: finish_owned<2>(a, recv, t, mt, ct, rank); break;
        case 4: finish_owned<4>(a, recv, t, mt, ct, rank); break;
        case 8: finish_owned<8>(a, recv, t, mt, ct, rank); break;
        default: finish_owned<16>(a, recv, t, mt, ct, rank); break;
        }
    }
    __syncthreads();                         // with peers: orders the storing threads' writes before thread 0's fence
    if (a.peers && threadIdx.x == 0) peer_signal_done(a.peers, gridDim.x);
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

cudaError_t launch_wave_umma_cluster(const WaveGroupArgs &g, const UmmaDesc &d, const CUtensorMap &tmap, bool dependent_launch, int num_sms, cudaStream_t s) {
    const uint32_t S = g.splits;
    if (!(S == 1 || S == 2 || S == 4 || S == 8 || S == 16) || g.count == 0 || g.count > (uint32_t)kMaxGroupWaves || g.total_clusters == 0) return cudaErrorInvalidValue;
    const uint32_t ctas = g.total_clusters * S;
    const bool deep = false;                              // the 7-stage, one-CTA-per-SM variant lost to cluster placement stalls; kept for tuning
    (void)num_sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(kUmmaThreads, 1, 1);
    cfg.dynamicSmemBytes = smallwave::smem_bytes(deep ? 7 : 3);
    cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    int n = 0;
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = S; attrs[n].val.clusterDim.y = 1; attrs[n].val.clusterDim.z = 1;
    ++n;
    if (dependent_launch) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n;
    if (S > 8) {    // clusters of 16 need an explicit opt-in
        const cudaError_t e = deep ? cudaFuncSetAttribute(k44_wave_umma_cluster_kernel<7>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1)
                                   : cudaFuncSetAttribute(k44_wave_umma_cluster_kernel<3>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return e;
    }
    return deep ? cudaLaunchKernelEx(&cfg, k44_wave_umma_cluster_kernel<7>, tmap, g, d)
                : cudaLaunchKernelEx(&cfg, k44_wave_umma_cluster_kernel<3>, tmap, g, d);
}

cudaError_t umma_kernel_setup() {
    cudaError_t e;
    if ((e = umma_setup_n64()) != cudaSuccess) return e;
    if ((e = umma_setup_n128()) != cudaSuccess) return e;
    if ((e = umma_setup_n256()) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(k44_wave_umma_cluster_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smallwave::smem_bytes(3))) != cudaSuccess) return e;
    return cudaFuncSetAttribute(k44_wave_umma_cluster_kernel<7>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smallwave::smem_bytes(7));
}

// ---------------------------------------------------------------------------------------------------
// packer kernels: one thread per 16-byte destination vector
// ---------------------------------------------------------------------------------------------------
template <int SRC>   // 0: container (16x16-tile) order, 1: row-major
__global__ void k44_repack_to_tiled_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, uint32_t cout,
                                           uint32_t fan_in, uint32_t num_kstages, uint64_t total) {
    for (uint64_t v = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; v < total; v += (uint64_t)gridDim.x * blockDim.x) {
        // invert tiled_vec_index: v = ((mt*KS + ks)*128 + r)*8 + pos
        const uint32_t pos = (uint32_t)(v & 7u), r = (uint32_t)((v >> 3) & 127u);
        const uint64_t blk = v >> 10;
        const uint32_t ks = (uint32_t)(blk % num_kstages), mt = (uint32_t)(blk / num_kstages);
        const uint32_t j = mt * 128u + r, k8 = ks * 8u + (pos ^ (r & 7u));
        uint4 val = make_uint4(0, 0, 0, 0);
        if (j < cout && k8 * 8u < fan_in) {
            const uint64_t si = SRC == 0 ? (((uint64_t)(j >> 4) * (fan_in >> 4) + (k8 >> 1)) * 32u + ((k8 & 1u) << 4) + (j & 15u))
                                         : ((uint64_t)j * (fan_in >> 3) + k8);
            val = src[si];
        }
        dst[v] = val;
    }
}

static inline uint32_t grid_for(uint64_t total, int block) {
    const uint64_t g = (total + block - 1) / block;
    return (uint32_t)(g < 148ull * 16ull ? (g ? g : 1) : 148ull * 16ull);
}

cudaError_t launch_repack_wmma_to_tiled(const uint4 *src, uint4 *dst, uint32_t cout, uint32_t fan_in, cudaStream_t s) {
    const uint32_t ks = (fan_in + kStageK - 1) / kStageK, mt = (cout + kTileM - 1) / kTileM;
    const uint64_t total = (uint64_t)mt * ks * 1024u;
    k44_repack_to_tiled_kernel<0><<<grid_for(total, 256), 256, 0, s>>>(src, dst, cout, fan_in, ks, total);
    return cudaGetLastError();
}

cudaError_t launch_repack_rowmajor_to_tiled(const uint4 *src, uint4 *dst, uint32_t cout, uint32_t fan_in, cudaStream_t s) {
    const uint32_t ks = (fan_in + kStageK - 1) / kStageK, mt = (cout + kTileM - 1) / kTileM;
    const uint64_t total = (uint64_t)mt * ks * 1024u;
    k44_repack_to_tiled_kernel<1><<<grid_for(total, 256), 256, 0, s>>>(src, dst, cout, fan_in, ks, total);
    return cudaGetLastError();
}

__global__ void k44_tiled_to_rowmajor_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, uint32_t fan_in,
                                             uint32_t num_kstages, uint64_t total) {
    const uint32_t v8 = fan_in >> 3;
    for (uint64_t v = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; v < total; v += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t j = (uint32_t)(v / v8), k8 = (uint32_t)(v % v8);
        dst[v] = src[tiled_vec_index(j, k8, num_kstages)];
    }
}

cudaError_t launch_tiled_to_rowmajor(const uint4 *src, uint4 *dst, uint32_t cout, uint32_t fan_in, cudaStream_t s) {
    const uint32_t ks = (fan_in + kStageK - 1) / kStageK;
    const uint64_t total = (uint64_t)cout * (fan_in >> 3);
    k44_tiled_to_rowmajor_kernel<<<grid_for(total, 256), 256, 0, s>>>(src, dst, fan_in, ks, total);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------
// host-I/O helpers: dense F32 [rows][width] <-> canvas rows (FP16, row pitch), on the device
// (the reference does this on the host: wavec/k44_wave_executor.cu:146-176)
// ---------------------------------------------------------------------------------------------------
__global__ void k44_f32_to_canvas_kernel(const float *__restrict__ src, __half *__restrict__ dst, uint32_t width,
                                         uint32_t pitch, uint64_t total) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / pitch;
        const uint32_t col = (uint32_t)(i % pitch);
        dst[i] = __float2half_rn(col < width ? src[row * width + col] : 0.0f);
    }
}

__global__ void k44_canvas_to_f32_kernel(const __half *__restrict__ src, float *__restrict__ dst, uint32_t width,
                                         uint32_t pitch, uint64_t total) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t row = i / width;
        const uint32_t col = (uint32_t)(i % width);
        dst[i] = __half2float(src[row * pitch + col]);
    }
}

cudaError_t launch_f32_to_canvas(const float *src, __half *dst, uint32_t rows, uint32_t width, uint32_t pitch, cudaStream_t s) {
    const uint64_t total = (uint64_t)rows * pitch;
    k44_f32_to_canvas_kernel<<<grid_for(total, 256), 256, 0, s>>>(src, dst, width, pitch, total);
    return cudaGetLastError();
}

cudaError_t launch_canvas_to_f32(const __half *src, float *dst, uint32_t rows, uint32_t width, uint32_t pitch, cudaStream_t s) {
    const uint64_t total = (uint64_t)rows * width;
    k44_canvas_to_f32_kernel<<<grid_for(total, 256), 256, 0, s>>>(src, dst, width, pitch, total);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------
// counter-based normal fill (synthetic weights of plans too large to generate on the host)
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__global__ void k44_fill_normal_f16_kernel(__half *dst, uint64_t n, uint64_t seed, float scale) {
    // each thread produces one Box-Muller pair
    for (uint64_t p = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; 2 * p < n; p += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t h = mix64(seed ^ (p * 0xD1342543DE82EF95ull));
        const float u1 = ((uint32_t)(h >> 40) + 1u) * (1.0f / 16777217.0f);      // (0,1]
        const float u2 = (uint32_t)(h & 0xffffffu) * (1.0f / 16777216.0f);
        const float rad = sqrtf(-2.0f * __logf(u1)) * scale;
        float sn, cs;
        __sincosf(6.28318530718f * u2, &sn, &cs);
        dst[2 * p] = __float2half_rn(rad * cs);
        if (2 * p + 1 < n) dst[2 * p + 1] = __float2half_rn(rad * sn);
    }
}

cudaError_t launch_fill_normal_f16(__half *dst, uint64_t n, uint64_t seed, float scale, cudaStream_t s) {
    k44_fill_normal_f16_kernel<<<grid_for((n + 1) / 2, 256), 256, 0, s>>>(dst, n, seed, scale);
    return cudaGetLastError();
}

}  // namespace k44b
