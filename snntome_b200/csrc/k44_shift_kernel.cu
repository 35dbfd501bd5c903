// Receptive-field token shift on the tensor cores (sm_100a).
//
// A shifted run reads its substrate rows `shift` columns (tokens) earlier: operand element (k, c) of a tile that
// starts at column t0 is canvas[row_k][t0 + c - shift], and zero where the column's position inside its frame
// is below the shift. A shift of 1..7 FP16 elements is not a legal start for a tensor copy (16-byte rule) and
// not a legal operand offset for tcgen05.mma, so the rows are realigned on their way into shared memory:
//
//   warp 0      streams, per 64-synapse step, the packed weight block (bulk copy) and the aligned window
//               [t0 - 8, t0 + N) of the step's substrate rows (one tensor copy per run, no swizzle) into a ring of
//               load stages; the ring is deep enough to cover the memory latency;
//   warps 6-9   ("aligners", 16 rows each per step) read their rows of the window from shared memory, funnel-shift
//               them by the run's shift in registers and store the result into a second, short ring in the
//               128-byte-swizzled operand layout;
//   warp 1      issues tcgen05.mma on (weights of the load stage, operand stage) and releases both;
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

constexpr int kTabEntries = 128;                    // run-table entries of one item held in shared memory (fan-in up to 2048 with 16-row runs)

// A tile of N_TILE columns is cut into sub-windows of at most 128 columns; each sub-window has its own copy of the
// 8 columns to its left (a tensor copy is at most 256 elements wide) and its own set of four aligner warps.
template <int N_TILE>
struct Cfg {
    static constexpr int kColBlocks = N_TILE / 64;
    static constexpr int kSubCols = N_TILE < 128 ? N_TILE : 128;
    static constexpr int kSubs = N_TILE / kSubCols;
    static constexpr int kThreads = 192 + 128 * kSubs;
    static constexpr uint32_t kXBytes = (uint32_t)kColBlocks * kStageK * 128u;      // operand stage
    static constexpr uint32_t kRawPitch = (uint32_t)(kSubCols + 8) * 2u;            // bytes per window row (an odd number of 16-byte chunks)
    static constexpr uint32_t kSubRawBytes = kStageK * kRawPitch;                   // a multiple of 128
    static constexpr uint32_t kRawBytes = (uint32_t)kSubs * kSubRawBytes;
    static constexpr int kLoadStages = N_TILE == 64 ? 6 : (N_TILE == 128 ? 5 : 3);  // weights + windows
    static constexpr int kOpStages = N_TILE == 256 ? 2 : 3;                         // realigned operand
    static constexpr uint32_t kTmemCols = 2u * N_TILE;
    static constexpr uint32_t kOutStageBytes = 128u * 80u;
    static constexpr uint32_t kSmemBytes = 1024u + (uint32_t)kLoadStages * (kStageWBytes + kRawBytes) + (uint32_t)kOpStages * kXBytes + 256u + kOutStageBytes + 2u * kTabEntries * 4u;
    static constexpr int kOutChunks = kSubCols / 16;    // 16-byte chunks one aligner lane produces per row
};

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
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
__global__ void __launch_bounds__(Cfg<N_TILE>::kThreads, 1)
k44_wave_umma_shift_kernel(const __grid_constant__ CUtensorMap tmap, const WaveArgs a, const UmmaDesc d) {
    using C = Cfg<N_TILE>;
    constexpr int SL = C::kLoadStages, SB = C::kOpStages;
    constexpr int OC = C::kOutChunks;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_smem = smem_base;                                        // SL weight blocks
    const uint32_t x_smem = w_smem + (uint32_t)SL * kStageWBytes;             // SB operand stages (swizzled)
    const uint32_t raw_smem = x_smem + (uint32_t)SB * C::kXBytes;             // SL windows (plain rows)
    const uint32_t ctl = raw_smem + (uint32_t)SL * C::kRawBytes;
    const uint32_t lfull_bar = ctl, lempty_bar = ctl + 8u * SL;               // load ring
    const uint32_t bfull_bar = ctl + 16u * SL, bempty_bar = bfull_bar + 8u * SB;   // operand ring
    const uint32_t tfull_bar = bempty_bar + 8u * SB, tempty_bar = tfull_bar + 16u;
    uint8_t *ctl_ptr = smem_raw + (ctl - ptx::smem_addr(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(ctl_ptr + 16 * SL + 16 * SB + 32);
    volatile uint32_t *abort_word = tmem_slot + 1;
    volatile uint32_t *epi_ok = tmem_slot + 4;
    uint8_t *out_stage = ctl_ptr + 256;
    const uint32_t tab_smem = ctl + 256u + C::kOutStageBytes;                  // two run-table buffers of kTabEntries words

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tiles_n = a.num_col_tiles64 / C::kColBlocks;
    const uint32_t mtiles = (a.cout + kTileM - 1) / kTileM;
    const uint32_t total_items = mtiles * tiles_n;
    const uint32_t KS = a.num_kstages;
    const uint32_t boxes_per_stage = kStageK / a.box_h;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SL; ++s) {
            ptx::mbar_init(lfull_bar + 8u * s, 1);       // producer's arrival carrying the byte count
            ptx::mbar_init(lempty_bar + 8u * s, 1 + 4 * C::kSubs);   // MMA commit (weights) + the aligner warps (windows)
        }
        for (int s = 0; s < SB; ++s) {
            ptx::mbar_init(bfull_bar + 8u * s, 4 * C::kSubs);        // the aligner warps
            ptx::mbar_init(bempty_bar + 8u * s, 1);      // MMA commit
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
    // column-tile-major walk: item -> (column tile, neuron tile)
    auto decode = [&](uint32_t item, uint32_t &mt, uint32_t &ct) { ct = item / mtiles; mt = item % mtiles; };
    const uint32_t my_items = blockIdx.x < total_items ? (total_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;

    if (warp == 0) {
        // ---------------- producer: weights and substrate windows ----------------
        // One thread runs the whole issue loop (no warp-wide exchange per step); the run-table entries of an item are
        // copied into a small shared-memory table by the whole warp one item ahead, with asynchronous 4-byte copies.
        if (lane == 0) ptx::prefetch_tensormap(&tmap);
        const uint64_t pol = ptx::policy_evict_last();     // weights and this column window are re-read by other tiles
        uint32_t issued = 0;
        bool ok = true;
        const uint32_t per_item = KS * boxes_per_stage;                     // table entries one item consumes
        const bool use_tab = per_item <= (uint32_t)kTabEntries;
        auto prefetch_entries = [&](uint32_t it) {
            uint32_t mt, ct;
            decode(blockIdx.x + it * gridDim.x, mt, ct);
            const uint32_t *rows = a.gather + (uint64_t)(mt / a.mtiles_per_group) * a.boxes_per_group;
            for (uint32_t e = lane; e < per_item; e += 32u)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(tab_smem + ((it & 1u) * kTabEntries + e) * 4u), "l"(rows + e) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (use_tab && my_items) prefetch_entries(0u);
        for (uint32_t it = 0; it < my_items; ++it) {
            if (use_tab) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncwarp();
                if (it + 1u < my_items) prefetch_entries(it + 1u);
            }
            // lane b issues box b of every step (issuing a tensor copy costs the issuing thread of the order of a hundred
            // cycles, so the boxes of a step go out as one warp instruction); lane 0 also posts the byte count and the
            // weight copy. The lanes need no exchange: each reads its own table entry.
            if (lane < boxes_per_stage * (uint32_t)C::kSubs) {
                uint32_t mt, ct;
                decode(blockIdx.x + it * gridDim.x, mt, ct);
                const uint4 *wsrc = a.w_tiles + (uint64_t)mt * KS * (kStageWBytes / 16u);
                const uint32_t *rows = a.gather + (uint64_t)(mt / a.mtiles_per_group) * a.boxes_per_group;
                const uint32_t tab_it = tab_smem + (it & 1u) * (kTabEntries * 4u);
                const uint32_t pb = lane / (uint32_t)C::kSubs, psub = lane % (uint32_t)C::kSubs;   // this lane's box and sub-window
                const int32_t x0 = (int32_t)(ct * (uint32_t)N_TILE + psub * (uint32_t)C::kSubCols) - 8;   // columns left of the row start read as zero
                for (uint32_t ks = 0; ks < KS; ++ks, ++issued) {
                    const uint32_t stage = issued % SL, ph = (issued / SL) & 1u;
                    const uint32_t bi = ks * boxes_per_stage + pb;
                    uint32_t e;
                    if (use_tab) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e) : "r"(tab_it + bi * 4u) : "memory");
                    else e = __ldg(rows + bi);
                    ok = wait(lempty_bar + 8u * stage, ph ^ 1u);
                    if (!ok) break;
                    if (lane == 0) {
                        ptx::mbar_arrive_expect_tx(lfull_bar + 8u * stage, kStageWBytes + C::kRawBytes);
                        ptx::bulk_g2s(w_smem + stage * kStageWBytes, wsrc + (uint64_t)ks * (kStageWBytes / 16u), kStageWBytes,
                                      lfull_bar + 8u * stage, pol);
                    }
                    ptx::tma_load_2d(raw_smem + stage * C::kRawBytes + psub * C::kSubRawBytes + pb * a.box_h * C::kRawPitch, &tmap, x0, (int32_t)(e & kBoxRowMask),
                                             lfull_bar + 8u * stage, pol);
                }
            }
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
            issued = __shfl_sync(0xffffffffu, issued, 0);
            if (!ok) break;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
            *abort_word = 1u;
            // wait (bounded) for copies already in flight before this CTA's shared memory goes away
            const uint32_t first = issued > (uint32_t)SL ? issued - SL : 0u;
            for (uint32_t i = first; i < issued; ++i) {
                const long long t0 = clock64();
                bool done = false;
                while (!done && (unsigned long long)(clock64() - t0) < d.wait_cycles)
                    done = ptx::mbar_try_wait(lfull_bar + 8u * (i % SL), (i / SL) & 1u);
                if (!done) atomicOr(a.status, (uint32_t)ST_TIMEOUT_DRAIN);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t it = 0; it < my_items && ok; ++it) {
                const uint32_t acc = it & 1u;
                ok = wait(tempty_bar + 8u * acc, ((it >> 1) & 1u) ^ 1u);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * N_TILE;
                for (uint32_t ks = 0; ks < KS; ++ks, ++g) {
                    const uint32_t ls = g % SL, lph = (g / SL) & 1u, bs = g % SB, bph = (g / SB) & 1u;
                    ok = wait(bfull_bar + 8u * bs, bph);                                      // operand realigned
                    ok = ok && wait(lfull_bar + 8u * ls, lph);                                // weights landed
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint64_t a0 = d.a_base | (uint64_t)(((w_smem + ls * kStageWBytes) >> 4) & 0x3fffu);
                    const uint64_t b0 = d.b_base | (uint64_t)(((x_smem + bs * C::kXBytes) >> 4) & 0x3fffu);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kStageK / 16u; ++k4)
                        ptx::umma_f16(d_tmem, a0 + (uint64_t)(k4 * d.a_k_step), b0 + (uint64_t)(k4 * d.b_k_step), d.idesc,
                                      (ks != 0u || k4 != 0u) ? 1u : 0u);
                    ptx::umma_commit(lempty_bar + 8u * ls);     // weight block reusable once these MMAs retire
                    ptx::umma_commit(bempty_bar + 8u * bs);     // operand stage likewise
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
        const uint32_t sub = (warp - 6u) >> 2, sw = (warp - 6u) & 3u;    // this warp: rows 16*sw .. 16*sw + 15 of sub-window `sub`
        const uint32_t r = lane & 15u, half = lane >> 4;    // 8 consecutive rows per shared-memory phase: conflict-free both ways
        const uint32_t krow = 16u * sw + r;
        const uint32_t first_chunk = half * (uint32_t)OC;                // inside the sub-window
        const uint32_t out_chunk0 = sub * (uint32_t)(C::kSubCols / 8) + first_chunk;   // inside the tile row
        const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
        uint32_t g = 0;
        bool ok = true;
        // table entries (row | shift << 28) of this warp's run in steps 0..31 of an item, one per lane; the next item's
        // entries are fetched while the current item is processed
        auto fetch = [&](uint32_t it, uint32_t ks_base) -> uint32_t {
            uint32_t mt, ct;
            decode(blockIdx.x + it * gridDim.x, mt, ct);
            const uint32_t *rows = a.gather + (uint64_t)(mt / a.mtiles_per_group) * a.boxes_per_group;
            const uint32_t ks = ks_base + lane;
            return ks < KS ? __ldg(rows + (ks * kStageK + 16u * sw) / a.box_h) : 0u;
        };
        uint32_t tab_next = my_items ? fetch(0u, 0u) : 0u;
        for (uint32_t it = 0; it < my_items && ok; ++it) {
            uint32_t mt, ct;
            decode(blockIdx.x + it * gridDim.x, mt, ct);
            uint32_t tab = tab_next;
            if (it + 1u < my_items) tab_next = fetch(it + 1u, 0u);
            const bool frame_start = ((ct * (uint32_t)N_TILE + sub * (uint32_t)C::kSubCols) % flen) == 0u;   // the 8 columns to the left belong to another frame
            for (uint32_t ks = 0; ks < KS; ++ks, ++g) {
                if (ks != 0u && (ks & 31u) == 0u) tab = fetch(it, ks);         // fan-in above 2048: fetched on demand
                const uint32_t ls = g % SL, lph = (g / SL) & 1u, bs = g % SB, bph = (g / SB) & 1u;
                const uint32_t sh = __shfl_sync(0xffffffffu, tab, ks & 31u) >> 28;
                uint32_t okw = 1u;
                if (lane == 0) okw = (wait(lfull_bar + 8u * ls, lph) && wait(bempty_bar + 8u * bs, bph ^ 1u)) ? 1u : 0u;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0u;
                if (!ok) break;
                uint4 buf[OC + 1];
                const uint32_t src = raw_smem + ls * C::kRawBytes + sub * C::kSubRawBytes + krow * C::kRawPitch + first_chunk * 16u;
#pragma unroll
                for (int i = 0; i <= OC; ++i) buf[i] = lds_v4(src + 16u * (uint32_t)i);
                if (half == 0u && frame_start) buf[0] = make_uint4(0u, 0u, 0u, 0u);
                const uint32_t dst_row = x_smem + bs * C::kXBytes + krow * 128u;
                switch (sh) {
                case 0: shift_and_store<0, OC>(buf, dst_row, out_chunk0, krow); break;
                case 1: shift_and_store<1, OC>(buf, dst_row, out_chunk0, krow); break;
                case 2: shift_and_store<2, OC>(buf, dst_row, out_chunk0, krow); break;
                case 3: shift_and_store<3, OC>(buf, dst_row, out_chunk0, krow); break;
                case 4: shift_and_store<4, OC>(buf, dst_row, out_chunk0, krow); break;
                case 5: shift_and_store<5, OC>(buf, dst_row, out_chunk0, krow); break;
                case 6: shift_and_store<6, OC>(buf, dst_row, out_chunk0, krow); break;
                case 7: shift_and_store<7, OC>(buf, dst_row, out_chunk0, krow); break;
                default: shift_and_store<8, OC>(buf, dst_row, out_chunk0, krow); break;
                }
                ptx::fence_proxy_async();          // generic-proxy stores -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(bfull_bar + 8u * bs);
                    ptx::mbar_arrive(lempty_bar + 8u * ls);     // this warp's rows of the window are in registers / stored
                }
            }
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
static cudaError_t launch(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s) {
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
    k44_wave_umma_shift_kernel<N_TILE><<<grid, C::kThreads, C::kSmemBytes, s>>>(tmap, a, d);
    return cudaGetLastError();
}

}  // namespace shiftwave

cudaError_t launch_wave_umma_shift(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s) {
    if (a.gather_mode != GATHER_BOX || a.box_h < 16u || (kStageK % a.box_h) != 0u) return cudaErrorInvalidValue;
    const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
    if (flen % d.n_tile != 0u || a.num_col_tiles64 % (d.n_tile / 64u) != 0u) return cudaErrorInvalidValue;
    if ((kStageK / a.box_h) * (d.n_tile > 128u ? d.n_tile / 128u : 1u) > 32u) return cudaErrorInvalidValue;   // one producer lane per box
    switch (d.n_tile) {
    case 64: return shiftwave::launch<64>(a, d, tmap, num_sms, s);
    case 128: return shiftwave::launch<128>(a, d, tmap, num_sms, s);
    case 256: return shiftwave::launch<256>(a, d, tmap, num_sms, s);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace k44b
