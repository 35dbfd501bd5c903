// Receptive-field token shift on the tensor cores (sm_100a).
//
// A shifted run reads its substrate rows `shift` columns (tokens) earlier: operand element (k, c) of a tile that
// starts at column t0 is canvas[row_k][t0 + c - shift], and zero where the column's position inside its frame
// is below the shift. A shift of 1..7 FP16 elements is not a legal start for a tensor copy (16-byte rule) and
// not a legal operand offset for tcgen05.mma, so the rows are realigned on their way into shared memory:
//
//   warp 0      streams the packed weight blocks with bulk copies (as in the unshifted kernel);
//   warps 6-9   ("aligners", one 16-row run each per stage) load the aligned window [t0 - 8, t0 + N) of their rows
//               from global memory with 16-byte loads, funnel-shift it by the run's shift in registers and store
//               the result in the 128-byte-swizzled operand layout; loads for the next stage are issued before
//               the current one is written, so the global latency hides behind the pipeline;
//   warp 1      issues tcgen05.mma once the weights have landed and the four aligners have arrived;
//   warps 2-5   epilogue out of double-buffered tensor memory (shared with the unshifted kernel).
//
// Tiles are walked column-tile-major: all neuron tiles of one column window run together, so the wave's weights
// and that window of the substrate stay in L2 and only compulsory bytes come from HBM.
//
// Every wait is bounded; on expiry the kernel records a status bit, stops and frees its tensor memory.
// Semantics follow kernels/cuda/kernel44_cuda_pack.cuh:242-264 (token-shift gather) with the causal zero padding
// of kernels/rocm/kernel44_rocm_pack.cuh:238-281.
#include "k44_kernels.cuh"
#include "k44_epilogue.cuh"
#include "k44_ptx.cuh"

namespace k44b {
namespace shiftwave {

constexpr int kThreads = 320;

template <int N_TILE>
struct Cfg {
    static constexpr int kColBlocks = N_TILE / 64;
    static constexpr uint32_t kXBytes = (uint32_t)kColBlocks * kStageK * 128u;
    static constexpr uint32_t kStageBytes = kStageWBytes + kXBytes;
    static constexpr int kStages = N_TILE == 64 ? 8 : 6;
    static constexpr uint32_t kTmemCols = 2u * N_TILE;
    static constexpr uint32_t kOutStageBytes = 128u * 80u;
    static constexpr uint32_t kSmemBytes = 1024u + (uint32_t)kStages * kStageBytes + 256u + kOutStageBytes;
    static constexpr int kOutChunks = N_TILE / 16;      // 16-byte chunks one aligner lane produces per row
};

__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// The lane holds OC + 1 consecutive 16-byte chunks of one row, starting 8 columns left of its first output
// column. Output element e is input element e + 8 - SHIFT; for odd shifts two neighbouring words are funnelled.
template <int SHIFT, int OC>
__device__ __forceinline__ void shift_and_store(const uint4 (&raw)[OC + 1], uint32_t dst_row, uint32_t first_chunk, uint32_t krow) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(raw);
    constexpr int m = SHIFT >> 1;
#pragma unroll
    for (int i = 0; i < OC; ++i) {
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int oi = 4 * i + e;
            if (SHIFT & 1) o[e] = __funnelshift_r(w[3 - m + oi], w[4 - m + oi], 16);
            else o[e] = w[4 - m + oi];
        }
        const uint32_t gq = first_chunk + (uint32_t)i;             // chunk index inside the tile row
        const uint32_t addr = dst_row + (gq >> 3) * (kStageK * 128u) + (((gq & 7u) ^ (krow & 7u)) << 4);
        sts_v4(addr, o[0], o[1], o[2], o[3]);
    }
}

template <int N_TILE>
__global__ void __launch_bounds__(kThreads, 1)
k44_wave_umma_shift_kernel(const WaveArgs a, const UmmaDesc d) {
    using C = Cfg<N_TILE>;
    constexpr int STAGES = C::kStages;
    constexpr int OC = C::kOutChunks;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_smem = smem_base;
    const uint32_t x_smem = smem_base + (uint32_t)STAGES * kStageWBytes;
    const uint32_t ctl = x_smem + (uint32_t)STAGES * C::kXBytes;
    const uint32_t full_bar = ctl, empty_bar = ctl + 8u * STAGES;
    const uint32_t tfull_bar = ctl + 16u * STAGES, tempty_bar = tfull_bar + 16u;
    uint8_t *ctl_ptr = smem_raw + (ctl - ptx::smem_addr(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(ctl_ptr + 16 * STAGES + 32);
    volatile uint32_t *abort_word = tmem_slot + 1;
    volatile uint32_t *epi_ok = tmem_slot + 4;
    uint8_t *out_stage = ctl_ptr + 256;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tiles_n = a.num_col_tiles64 / C::kColBlocks;
    const uint32_t mtiles = (a.cout + kTileM - 1) / kTileM;
    const uint32_t total_items = mtiles * tiles_n;
    const uint32_t KS = a.num_kstages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar + 8u * s, 5);      // weight copy (with its byte count) + four aligner warps
            ptx::mbar_init(empty_bar + 8u * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar + 8u * b, 1);
            ptx::mbar_init(tempty_bar + 8u * b, 128);
        }
        *abort_word = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(const_cast<uint32_t *>(tmem_slot)), C::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto wait = [&](uint32_t bar, uint32_t parity) -> bool {
        const long long t0 = clock64();
        for (uint32_t it = 0;; ++it) {
            if (ptx::mbar_try_wait(bar, parity)) return true;
            if ((it & 31u) == 31u) {
                if (*abort_word != 0u) return false;
                if ((unsigned long long)(clock64() - t0) > d.wait_cycles) return false;
            }
        }
    };
    // column-tile-major walk: item -> (column tile, neuron tile)
    auto decode = [&](uint32_t item, uint32_t &mt, uint32_t &ct) { ct = item / mtiles; mt = item % mtiles; };
    const uint32_t my_items = blockIdx.x < total_items ? (total_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;

    if (warp == 0) {
        // ---------------- weight producer ----------------
        if (lane == 0) {
            const uint64_t pol_w = ptx::policy_evict_last();    // the wave's weights are re-read by every column tile
            uint32_t issued = 0;
            bool ok = true;
            for (uint32_t it = 0; it < my_items && ok; ++it) {
                uint32_t mt, ct;
                decode(blockIdx.x + it * gridDim.x, mt, ct);
                const uint4 *wsrc = a.w_tiles + (uint64_t)mt * KS * (kStageWBytes / 16u);
                for (uint32_t ks = 0; ks < KS; ++ks, ++issued) {
                    const uint32_t stage = issued % STAGES, ph = (issued / STAGES) & 1u;
                    ok = wait(empty_bar + 8u * stage, ph ^ 1u);
                    if (!ok) break;
                    ptx::mbar_arrive_expect_tx(full_bar + 8u * stage, kStageWBytes);
                    ptx::bulk_g2s(w_smem + stage * kStageWBytes, wsrc + (uint64_t)ks * (kStageWBytes / 16u), kStageWBytes,
                                  full_bar + 8u * stage, pol_w);
                }
            }
            if (!ok) {
                if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
                *abort_word = 1u;
                // the copies still in flight complete on barriers nobody may be waiting on any more: give them time
                const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0u;
                for (uint32_t i = first; i < issued; ++i) {
                    const long long t0 = clock64();
                    bool done = false;
                    while (!done && (unsigned long long)(clock64() - t0) < d.wait_cycles)
                        done = ptx::mbar_try_wait(full_bar + 8u * (i % STAGES), (i / STAGES) & 1u);
                    if (!done) atomicOr(a.status, (uint32_t)ST_TIMEOUT_DRAIN);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t consumed = 0;
            bool ok = true;
            for (uint32_t it = 0; it < my_items && ok; ++it) {
                const uint32_t acc = it & 1u;
                ok = wait(tempty_bar + 8u * acc, ((it >> 1) & 1u) ^ 1u);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * N_TILE;
                for (uint32_t ks = 0; ks < KS; ++ks, ++consumed) {
                    const uint32_t stage = consumed % STAGES, ph = (consumed / STAGES) & 1u;
                    ok = wait(full_bar + 8u * stage, ph);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint64_t a0 = d.a_base | (uint64_t)(((w_smem + stage * kStageWBytes) >> 4) & 0x3fffu);
                    const uint64_t b0 = d.b_base | (uint64_t)(((x_smem + stage * C::kXBytes) >> 4) & 0x3fffu);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kStageK / 16u; ++k4)
                        ptx::umma_f16(d_tmem, a0 + (uint64_t)(k4 * d.a_k_step), b0 + (uint64_t)(k4 * d.b_k_step), d.idesc,
                                      (ks != 0u || k4 != 0u) ? 1u : 0u);
                    ptx::umma_commit(empty_bar + 8u * stage);
                }
                if (ok) ptx::umma_commit(tfull_bar + 8u * acc);
            }
            if (!ok) {
                if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_MMA);
                *abort_word = 1u;
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ---------------- epilogue ----------------
        const uint32_t quarter = warp & 3u;
        const bool has_map = a.cout_map != nullptr;
        bool ok = true;
        for (uint32_t it = 0; it < my_items && ok; ++it) {
            uint32_t mt, ct;
            decode(blockIdx.x + it * gridDim.x, mt, ct);
            const uint32_t acc = it & 1u;
            if (threadIdx.x == 64u) epi_ok[it & 1u] = wait(tfull_bar + 8u * acc, (it >> 1) & 1u) ? 1u : 0u;
            epilogue_bar_sync();
            ok = epi_ok[it & 1u] != 0u;
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t j = mt * kTileM + quarter * 32u + lane;
            const bool live = j < a.cout;
            const uint32_t oj = (live && has_map) ? a.cout_map[j] : j;
            const float bias = (live && a.bias) ? __half2float(a.bias[j]) : 0.0f;
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < (uint32_t)N_TILE; c0 += 32u) {
                uint32_t v[32];
                ptx::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * N_TILE + c0, v);
                ptx::tmem_ld_wait();
                float f[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(v[e]);
                stage_and_store(a, f, bias, has_map, live, oj, (uint64_t)ct * N_TILE + c0, out_stage + quarter * (32u * 80u), lane);
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(tempty_bar + 8u * acc);
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_EPILOGUE);
            *abort_word = 1u;
        }
    } else {
        // ---------------- aligners ----------------
        const uint32_t sw = warp - 6u;                      // rows 16*sw .. 16*sw + 15 of every stage
        const uint32_t r = lane >> 1, half = lane & 1u;
        const uint32_t krow = 16u * sw + r;
        const uint32_t first_chunk = half * (uint32_t)OC;
        const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
        const uint32_t total = my_items * KS;

        uint4 bufA[OC + 1], bufB[OC + 1];
        uint32_t shA = 0, shB = 0;

        // issue the global loads of flattened step g (item g / KS, stage g % KS)
        auto load = [&](uint32_t g, uint4 (&buf)[OC + 1], uint32_t &sh) {
            uint32_t mt, ct;
            decode(blockIdx.x + (g / KS) * gridDim.x, mt, ct);
            const uint32_t ks = g % KS;
            const uint32_t k0 = ks * kStageK + 16u * sw;                   // first synapse of this warp's run
            const uint32_t *rows = a.gather + (uint64_t)(mt / a.mtiles_per_group) * a.boxes_per_group;
            const uint32_t e = __ldg(rows + k0 / a.box_h);
            sh = e >> 28;
            const uint32_t row = (e & kBoxRowMask) + (k0 % a.box_h) + r;
            const uint32_t t0 = ct * (uint32_t)N_TILE;
            const bool frame_start = (t0 % flen) == 0u;                    // the 8 columns left of the tile belong to another frame
            const __half *src = a.canvas + (uint64_t)row * a.pitch + t0 + first_chunk * 8u;
#pragma unroll
            for (int i = 0; i <= OC; ++i) {
                if (i == 0 && half == 0u && frame_start) buf[0] = make_uint4(0u, 0u, 0u, 0u);
                else buf[i] = ldg_nc_v4(src + 8 * i - 8);
            }
        };
        // realign and store step g into its pipeline stage, then arrive
        auto store = [&](uint32_t g, const uint4 (&buf)[OC + 1], uint32_t sh) -> bool {
            const uint32_t stage = g % STAGES, ph = (g / STAGES) & 1u;
            uint32_t ok = 1u;
            if (lane == 0) ok = wait(empty_bar + 8u * stage, ph ^ 1u) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) return false;
            const uint32_t dst_row = x_smem + stage * C::kXBytes + krow * 128u;
            switch (sh) {
            case 0: shift_and_store<0, OC>(buf, dst_row, first_chunk, krow); break;
            case 1: shift_and_store<1, OC>(buf, dst_row, first_chunk, krow); break;
            case 2: shift_and_store<2, OC>(buf, dst_row, first_chunk, krow); break;
            case 3: shift_and_store<3, OC>(buf, dst_row, first_chunk, krow); break;
            case 4: shift_and_store<4, OC>(buf, dst_row, first_chunk, krow); break;
            case 5: shift_and_store<5, OC>(buf, dst_row, first_chunk, krow); break;
            case 6: shift_and_store<6, OC>(buf, dst_row, first_chunk, krow); break;
            case 7: shift_and_store<7, OC>(buf, dst_row, first_chunk, krow); break;
            default: shift_and_store<8, OC>(buf, dst_row, first_chunk, krow); break;
            }
            ptx::fence_proxy_async();          // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(full_bar + 8u * stage);
            return true;
        };

        bool ok = true;
        if (total > 0u) load(0u, bufA, shA);
        for (uint32_t g = 0; g < total && ok; g += 2u) {
            if (g + 1u < total) load(g + 1u, bufB, shB);
            ok = store(g, bufA, shA);
            if (!ok) break;
            if (g + 2u < total) load(g + 2u, bufA, shA);
            if (g + 1u < total) ok = store(g + 1u, bufB, shB);
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
            *abort_word = 1u;
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

template <int N_TILE>
static cudaError_t launch(const WaveArgs &a, const UmmaDesc &d, int num_sms, cudaStream_t s) {
    using C = Cfg<N_TILE>;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        e = cudaFuncSetAttribute(k44_wave_umma_shift_kernel<N_TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const uint32_t mtiles = (a.cout + kTileM - 1) / kTileM;
    const uint32_t items = mtiles * (a.num_col_tiles64 / (N_TILE / 64u));
    const uint32_t grid = items < (uint32_t)num_sms ? items : (uint32_t)num_sms;
    k44_wave_umma_shift_kernel<N_TILE><<<grid, kThreads, C::kSmemBytes, s>>>(a, d);
    return cudaGetLastError();
}

}  // namespace shiftwave

cudaError_t launch_wave_umma_shift(const WaveArgs &a, const UmmaDesc &d, int num_sms, cudaStream_t s) {
    if (a.gather_mode != GATHER_BOX || a.box_h < 16u || (kStageK % a.box_h) != 0u) return cudaErrorInvalidValue;
    const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
    if (flen % d.n_tile != 0u || a.num_col_tiles64 % (d.n_tile / 64u) != 0u) return cudaErrorInvalidValue;
    switch (d.n_tile) {
    case 64: return shiftwave::launch<64>(a, d, num_sms, s);
    case 128: return shiftwave::launch<128>(a, d, num_sms, s);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace k44b
