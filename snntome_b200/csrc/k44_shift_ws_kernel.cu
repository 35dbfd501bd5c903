// Receptive-field token shift on the tensor cores with the weights held in tensor memory (sm_100a).
//
// In the token-shift kernel of k44_shift_kernel.cu every byte of the realigned operand crosses shared memory four times per
// 64-synapse step (window written by the tensor copy, read by the aligners, written back realigned, read by the MMA) and the
// weight block twice (written by the bulk copy, read by the MMA), each with its own barrier round trip.
// A wave whose fan-in is at most 512 has weight tiles of 128 neurons x 512 synapses = 128 KiB, which fit 256 of the 512
// tensor-memory columns as the A operand of tcgen05.mma. This kernel therefore makes a work item one neuron tile times a
// run of consecutive column tiles: the weight tile is copied shared memory -> tensor memory once per item (tcgen05.cp
// 128x256b out of the same packed blocks the streaming kernels use), and every MMA of the item reads A from tensor memory,
// so that in the steady state shared memory carries the substrate operand only.
//
//   warp 0        per item: the 16 KiB weight blocks of the neuron tile (bulk copies into a two-block ring), then per column
//                 tile and ring stage (two 64-synapse steps) the aligned windows [t0 - 8, t0 + 128) of the stage's substrate
//                 rows (one tensor copy per run, one lane per copy);
//   warp 1        one thread: tcgen05.cp of the weight blocks while the item's first column tile runs, tcgen05.mma (A in tensor
//                 memory, B = operand ring, M 128 x N 128 x K 16, eight per stage) into one of two accumulators;
//   warps 2-5, 6-9  epilogue out of tensor memory, one group per 64-column half of the tile, overlapping the next tile;
//   warps 10..    ("aligners", AG groups of four warps) realign the window rows by the run's shift into the 128-byte-swizzled
//                 operand ring; group g takes the stages g, g + AG, ...
//
// Why the roles look like this: a role that is one warp issues an instruction every ~9 cycles, so what bounds such a pipeline
// is the number of barrier round trips and instructions per role and step, not bytes. Hence two steps per stage, a first
// barrier try before the clock is read for the bounded wait, whole-warp waits in the aligners, and two groups for each of the
// two roles with real arithmetic (with one epilogue group the GELU of a 128 x 128 tile took longer than the tile's MMAs).
//
// Items are numbered column-run-major, so that the CTAs working at the same time read the same columns of the substrate
// and share them through L2. Every wait is bounded; on expiry the kernel records a status bit, stops and frees its tensor
// memory. Semantics as in k44_shift_kernel.cu (kernels/cuda/kernel44_cuda_pack.cuh:242-264, causal zero padding of
// kernels/rocm/kernel44_rocm_pack.cuh:238-281).
#include "k44_kernels.cuh"
#include "k44_epilogue.cuh"
#include "k44_ptx.cuh"

namespace k44b {
namespace shiftws {

constexpr int kN = 128;                             // columns per tile
constexpr int kTabEntries = 32;                     // run-table entries of one item (fan-in 512 in 16-row runs)
constexpr int kMaxKS = 8;                           // 64-synapse steps whose weights fit tensor memory
constexpr int kSub = 2;                             // 64-synapse steps per ring stage: one barrier round trip serves two of them
constexpr int SL = 3, SB = 2, SW = 2;               // window ring, operand ring, weight ring (blocks of one step); 2 + 3 instead of 3 + 2 was 10 % slower
constexpr uint32_t kXBytes = 2u * kStageK * 128u;                // operand of one step: two 64-column blocks
constexpr uint32_t kRawPitch = (uint32_t)(kN + 8) * 2u;          // bytes per window row (17 chunks of 16 bytes)
constexpr uint32_t kRawBytes = kStageK * kRawPitch;              // window of one step
constexpr uint32_t kXStage = kSub * kXBytes, kRawStage = kSub * kRawBytes;
constexpr uint32_t kTmemCols = 512u;                             // accumulators at columns 0 / 128, weights at 256..511
constexpr uint32_t kATmemCol = 256u;
constexpr uint32_t kOutStageBytes = 2u * 128u * 80u;            // one padded slot per epilogue thread
constexpr int kFirstAligner = 10;                   // warps 0 producer, 1 MMA, 2-5 and 6-9 epilogue, 10.. aligners
constexpr uint32_t kSmemBytes = 1024u + (uint32_t)SL * kRawStage + (uint32_t)SB * kXStage + (uint32_t)SW * kStageWBytes + 256u + kOutStageBytes + 2u * kTabEntries * 4u;
constexpr int OC = kN / 16;                         // 16-byte chunks one aligner lane produces per row

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// The lane holds OC + 1 consecutive 16-byte chunks of one row, starting 8 columns left of its first output column.
// Output element e is input element e + 8 - SHIFT; for odd shifts two neighbouring words are funnelled.
template <int SHIFT>
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
        const uint32_t gq = first_chunk + (uint32_t)i;
        sts_v4(dst_row + (gq >> 3) * (kStageK * 128u) + (((gq & 7u) ^ (krow & 7u)) << 4), o[0], o[1], o[2], o[3]);
    }
}

template <int AG>
__global__ void __launch_bounds__(32 * kFirstAligner + 128 * AG, 1)
k44_wave_umma_shift_ws_kernel(const __grid_constant__ CUtensorMap tmap, const WaveArgs a, const UmmaDesc d) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_smem = smem_base;                                        // SW weight blocks
    const uint32_t x_smem = w_smem + (uint32_t)SW * kStageWBytes;             // SB operand stages (swizzled)
    const uint32_t raw_smem = x_smem + (uint32_t)SB * kXStage;                // SL windows (plain rows)
    const uint32_t ctl = raw_smem + (uint32_t)SL * kRawStage;
    const uint32_t lfull_bar = ctl, lempty_bar = lfull_bar + 8u * SL;         // window ring
    const uint32_t bfull_bar = lempty_bar + 8u * SL, bempty_bar = bfull_bar + 8u * SB;   // operand ring
    const uint32_t wfull_bar = bempty_bar + 8u * SB, wempty_bar = wfull_bar + 8u * SW;   // weight ring
    const uint32_t tfull_bar = wempty_bar + 8u * SW, tempty_bar = tfull_bar + 16u;
    const uint32_t adone_bar = tempty_bar + 16u;                              // every MMA of an item has retired: its weights may be replaced
    uint8_t *ctl_ptr = smem_raw + (ctl - ptx::smem_addr(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(ctl_ptr + 16 * SL + 16 * SB + 16 * SW + 40);
    volatile uint32_t *abort_word = tmem_slot + 1;
    volatile uint32_t *epi_ok = tmem_slot + 2;             // [group][tile parity]
    uint8_t *out_stage = ctl_ptr + 256;
    const uint32_t tab_smem = ctl + 256u + kOutStageBytes;                    // two run-table buffers of kTabEntries words

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tiles_n = a.num_col_tiles64 / 2u;
    const uint32_t mtiles = (a.cout + kTileM - 1) / kTileM;
    const uint32_t chunk = d.ws_chunk;                                         // column tiles per item
    const uint32_t chunks = (tiles_n + chunk - 1u) / chunk;
    const uint32_t total_items = mtiles * chunks;
    const uint32_t KS = a.num_kstages;
    const uint32_t ST = (KS + (uint32_t)kSub - 1u) / (uint32_t)kSub;           // ring stages per tile
    const uint32_t boxes_per_step = kStageK / a.box_h;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SL; ++s) {
            ptx::mbar_init(lfull_bar + 8u * s, 1);
            ptx::mbar_init(lempty_bar + 8u * s, 4);      // the aligner warps
        }
        for (int s = 0; s < SB; ++s) {
            ptx::mbar_init(bfull_bar + 8u * s, 4);
            ptx::mbar_init(bempty_bar + 8u * s, 1);      // MMA commit
        }
        for (int s = 0; s < SW; ++s) {
            ptx::mbar_init(wfull_bar + 8u * s, 1);
            ptx::mbar_init(wempty_bar + 8u * s, 1);      // commit behind the copies to tensor memory
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar + 8u * b, 1);
            ptx::mbar_init(tempty_bar + 8u * b, 256);
        }
        ptx::mbar_init(adone_bar, 1);
        *abort_word = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
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
    // item -> neuron tile and run of column tiles [ct0, ct1)
    auto decode = [&](uint32_t item, uint32_t &mt, uint32_t &ct0, uint32_t &ct1) {
        const uint32_t c = item / mtiles;
        mt = item % mtiles;
        ct0 = c * chunk;
        ct1 = ct0 + chunk < tiles_n ? ct0 + chunk : tiles_n;
    };
    const uint32_t my_items = blockIdx.x < total_items ? (total_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    const uint32_t per_item = KS * boxes_per_step;                             // table entries of one item (<= kTabEntries, checked by the launcher)

    if (warp == 0) {
        // ---------------- producer: weights once per item, substrate windows per tile ----------------
        if (lane == 0) ptx::prefetch_tensormap(&tmap);
        const uint64_t pol = ptx::policy_evict_last();
        uint32_t issued = 0, wissued = 0;
        bool ok = true;
        auto prefetch_entries = [&](uint32_t it) {
            uint32_t mt, c0, c1;
            decode(blockIdx.x + it * gridDim.x, mt, c0, c1);
            const uint32_t *rows = a.gather + (uint64_t)(mt / a.mtiles_per_group) * a.boxes_per_group;
            for (uint32_t e = lane; e < per_item; e += 32u)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(tab_smem + ((it & 1u) * kTabEntries + e) * 4u), "l"(rows + e) : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        if (my_items) prefetch_entries(0u);
        for (uint32_t it = 0; it < my_items; ++it) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
            if (it + 1u < my_items) prefetch_entries(it + 1u);
            if (lane < (uint32_t)kSub * boxes_per_step) {       // lane b issues box b of every stage; lane 0 also the weights and the byte counts
                uint32_t mt, ct0, ct1;
                decode(blockIdx.x + it * gridDim.x, mt, ct0, ct1);
                const uint4 *wsrc = a.w_tiles + (uint64_t)mt * KS * (kStageWBytes / 16u);
                const uint32_t tab_it = tab_smem + (it & 1u) * (kTabEntries * 4u);
                for (uint32_t ct = ct0; ct < ct1 && ok; ++ct) {
                    const int32_t x0 = (int32_t)(ct * (uint32_t)kN) - 8;          // columns left of the row start read as zero
                    for (uint32_t st = 0; st < ST; ++st, ++issued) {
                        const uint32_t nsub = min((uint32_t)kSub, KS - st * (uint32_t)kSub);
                        if (ct == ct0 && lane == 0) {
                            for (uint32_t sb = 0; sb < nsub && ok; ++sb, ++wissued) {
                                const uint32_t ws = wissued % SW, wph = (wissued / SW) & 1u;
                                ok = wait(wempty_bar + 8u * ws, wph ^ 1u);
                                if (ok) {
                                    ptx::mbar_arrive_expect_tx(wfull_bar + 8u * ws, kStageWBytes);
                                    ptx::bulk_g2s(w_smem + ws * kStageWBytes, wsrc + (uint64_t)(st * kSub + sb) * (kStageWBytes / 16u), kStageWBytes, wfull_bar + 8u * ws, pol);
                                }
                            }
                        }
                        const uint32_t stage = issued % SL, ph = (issued / SL) & 1u;
                        const bool mine = lane < nsub * boxes_per_step;
                        uint32_t e = 0;
                        if (mine) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e) : "r"(tab_it + (st * (uint32_t)kSub * boxes_per_step + lane) * 4u) : "memory");
                        ok = ok && wait(lempty_bar + 8u * stage, ph ^ 1u);
                        if (!ok) break;
                        if (lane == 0) ptx::mbar_arrive_expect_tx(lfull_bar + 8u * stage, nsub * kRawBytes);
                        if (mine) ptx::tma_load_2d(raw_smem + stage * kRawStage + lane * a.box_h * kRawPitch, &tmap, x0, (int32_t)(e & kBoxRowMask), lfull_bar + 8u * stage, pol);
                    }
                }
            }
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
            issued = __shfl_sync(0xffffffffu, issued, 0);
            wissued = __shfl_sync(0xffffffffu, wissued, 0);       // (only lane 0 counts weight blocks)
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
                while (!done && (unsigned long long)(clock64() - t0) < d.wait_cycles) done = ptx::mbar_try_wait(lfull_bar + 8u * (i % SL), (i / SL) & 1u);
                if (!done) atomicOr(a.status, (uint32_t)ST_TIMEOUT_DRAIN);
            }
            const uint32_t wfirst = wissued > (uint32_t)SW ? wissued - SW : 0u;
            for (uint32_t i = wfirst; i < wissued; ++i) {
                const long long t0 = clock64();
                bool done = false;
                while (!done && (unsigned long long)(clock64() - t0) < d.wait_cycles) done = ptx::mbar_try_wait(wfull_bar + 8u * (i % SW), (i / SW) & 1u);
                if (!done) atomicOr(a.status, (uint32_t)ST_TIMEOUT_DRAIN);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- weights into tensor memory, MMA issue ----------------
        if (lane == 0) {
            uint32_t g = 0, wg = 0, tc = 0;
            bool ok = true;
            const uint32_t a_tmem = tmem_base + kATmemCol;
            for (uint32_t it = 0; it < my_items && ok; ++it) {
                uint32_t mt, ct0, ct1;
                decode(blockIdx.x + it * gridDim.x, mt, ct0, ct1);
                // the previous item's MMAs still read its weights: replace them only when all of them have retired
                if (it != 0u) ok = wait(adone_bar, (it - 1u) & 1u);
                for (uint32_t ct = ct0; ct < ct1 && ok; ++ct, ++tc) {
                    const uint32_t acc = tc & 1u;
                    ok = wait(tempty_bar + 8u * acc, ((tc >> 1) & 1u) ^ 1u);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * kN;
                    for (uint32_t st = 0; st < ST; ++st, ++g) {
                        const uint32_t nsub = min((uint32_t)kSub, KS - st * (uint32_t)kSub);
                        if (ct == ct0) {
                            for (uint32_t sb = 0; sb < nsub && ok; ++sb, ++wg) {
                                const uint32_t ws = wg % SW, wph = (wg / SW) & 1u, ks = st * (uint32_t)kSub + sb;
                                ok = wait(wfull_bar + 8u * ws, wph);
                                if (!ok) break;
                                ptx::tc_fence_after();
                                const uint64_t a0 = d.a_base | (uint64_t)(((w_smem + ws * kStageWBytes) >> 4) & 0x3fffu);
#pragma unroll
                                for (uint32_t k4 = 0; k4 < kStageK / 16u; ++k4)
                                    ptx::tmem_cp_128x256b(a_tmem + ks * 32u + k4 * 8u, a0 + (uint64_t)(k4 * d.a_k_step));
                                ptx::umma_commit(wempty_bar + 8u * ws);       // block reusable once the copies have read it
                            }
                            if (!ok) break;
                        }
                        const uint32_t bs = g % SB, bph = (g / SB) & 1u;
                        ok = wait(bfull_bar + 8u * bs, bph);
                        if (!ok) break;
                        ptx::tc_fence_after();
                        for (uint32_t sb = 0; sb < nsub; ++sb) {
                            const uint32_t ks = st * (uint32_t)kSub + sb;
                            const uint64_t b0 = d.b_base | (uint64_t)(((x_smem + bs * kXStage + sb * kXBytes) >> 4) & 0x3fffu);
#pragma unroll
                            for (uint32_t k4 = 0; k4 < kStageK / 16u; ++k4)
                                ptx::umma_f16_a_tmem(d_tmem, a_tmem + ks * 32u + k4 * 8u, b0 + (uint64_t)(k4 * d.b_k_step), d.idesc, (ks != 0u || k4 != 0u) ? 1u : 0u);
                        }
                        ptx::umma_commit(bempty_bar + 8u * bs);
                    }
                    if (ok) ptx::umma_commit(tfull_bar + 8u * acc);
                }
                if (ok) ptx::umma_commit(adone_bar);
            }
            if (!ok) {
                if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_MMA);
                *abort_word = 1u;
            }
        }
        __syncwarp();
    } else if (warp < (uint32_t)kFirstAligner) {
        // ---------------- epilogue: two groups of four warps, 64 columns of every tile each ----------------
        // (one warp per scheduler and group: a lone warp issues an instruction every several cycles, and at fan-in 512 the
        // epilogue of a GELU wave costs more issue time than the tile's MMAs — one group alone bounded the kernel)
        const uint32_t quarter = warp & 3u, eg = (warp - 2u) >> 2;
        const uint32_t first_thread = 64u + 128u * eg;
        const bool has_map = a.cout_map != nullptr;
        bool ok = true;
        uint32_t tc = 0;
        for (uint32_t it = 0; it < my_items && ok; ++it) {
            uint32_t mt, ct0, ct1;
            decode(blockIdx.x + it * gridDim.x, mt, ct0, ct1);
            const uint32_t j = mt * kTileM + quarter * 32u + lane;
            const bool live = j < a.cout;
            const uint32_t oj = (live && has_map) ? a.cout_map[j] : j;
            const float bias = (live && a.bias) ? __half2float(a.bias[j]) : 0.0f;
            for (uint32_t ct = ct0; ct < ct1 && ok; ++ct, ++tc) {
                const uint32_t acc = tc & 1u;
                if (threadIdx.x == first_thread) epi_ok[2u * eg + (tc & 1u)] = wait(tfull_bar + 8u * acc, (tc >> 1) & 1u) ? 1u : 0u;
                asm volatile("bar.sync %0, 128;" ::"r"(1u + eg) : "memory");
                ok = epi_ok[2u * eg + (tc & 1u)] != 0u;
                if (!ok) break;
                ptx::tc_fence_after();
#pragma unroll 1
                for (uint32_t c0 = 64u * eg; c0 < 64u * eg + 64u; c0 += 32u) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * kN + c0, v);
                    ptx::tmem_ld_wait();
                    float f[32];
#pragma unroll
                    for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(v[e]);
                    stage_and_store(a, f, bias, has_map, live, oj, (uint64_t)ct * kN + c0, out_stage + (4u * eg + quarter) * (32u * 80u), lane);
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(tempty_bar + 8u * acc);
            }
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_EPILOGUE);
            *abort_word = 1u;
        }
    } else {
        // ---------------- aligners ----------------
        const uint32_t sw = (warp - (uint32_t)kFirstAligner) & 3u;               // this warp: rows 16*sw .. 16*sw + 15 of every window of its group's steps
        const uint32_t grp = (warp - (uint32_t)kFirstAligner) >> 2;
        const uint32_t r = lane & 15u, half = lane >> 4;    // 8 consecutive rows per shared-memory phase: conflict-free both ways
        const uint32_t krow = 16u * sw + r;
        const uint32_t first_chunk = half * (uint32_t)OC;
        const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
        uint32_t g = 0;
        bool ok = true;
        // table entries (row | shift << 28) of this warp's run in the steps of an item, one per lane
        auto fetch = [&](uint32_t it) -> uint32_t {
            uint32_t mt, c0, c1;
            decode(blockIdx.x + it * gridDim.x, mt, c0, c1);
            const uint32_t *rows = a.gather + (uint64_t)(mt / a.mtiles_per_group) * a.boxes_per_group;
            return lane < KS ? __ldg(rows + (lane * kStageK + 16u * sw) / a.box_h) : 0u;
        };
        uint32_t tab_next = my_items ? fetch(0u) : 0u;
        for (uint32_t it = 0; it < my_items && ok; ++it) {
            uint32_t mt, ct0, ct1;
            decode(blockIdx.x + it * gridDim.x, mt, ct0, ct1);
            const uint32_t tab = tab_next;
            if (it + 1u < my_items) tab_next = fetch(it + 1u);
            for (uint32_t ct = ct0; ct < ct1 && ok; ++ct) {
                const bool frame_start = ((ct * (uint32_t)kN) % flen) == 0u;     // the 8 columns to the left belong to another frame
                for (uint32_t st = 0; st < ST; ++st, ++g) {
                    if (AG > 1 && g % (uint32_t)AG != grp) continue;
                    const uint32_t nsub = min((uint32_t)kSub, KS - st * (uint32_t)kSub);
                    const uint32_t ls = g % SL, lph = (g / SL) & 1u, bs = g % SB, bph = (g / SB) & 1u;
                    ok = __all_sync(0xffffffffu, (wait(lfull_bar + 8u * ls, lph) && wait(bempty_bar + 8u * bs, bph ^ 1u)) ? 1 : 0) != 0;
                    if (!ok) break;
                    for (uint32_t sb = 0; sb < nsub; ++sb) {
                        const uint32_t sh = __shfl_sync(0xffffffffu, tab, st * (uint32_t)kSub + sb) >> 28;
                        uint4 buf[OC + 1];
                        const uint32_t src = raw_smem + ls * kRawStage + sb * kRawBytes + krow * kRawPitch + first_chunk * 16u;
#pragma unroll
                        for (int i = 0; i <= OC; ++i) buf[i] = lds_v4(src + 16u * (uint32_t)i);
                        if (half == 0u && frame_start) buf[0] = make_uint4(0u, 0u, 0u, 0u);
                        const uint32_t dst_row = x_smem + bs * kXStage + sb * kXBytes + krow * 128u;
                        switch (sh) {
                        case 0: shift_and_store<0>(buf, dst_row, first_chunk, krow); break;
                        case 1: shift_and_store<1>(buf, dst_row, first_chunk, krow); break;
                        case 2: shift_and_store<2>(buf, dst_row, first_chunk, krow); break;
                        case 3: shift_and_store<3>(buf, dst_row, first_chunk, krow); break;
                        case 4: shift_and_store<4>(buf, dst_row, first_chunk, krow); break;
                        case 5: shift_and_store<5>(buf, dst_row, first_chunk, krow); break;
                        case 6: shift_and_store<6>(buf, dst_row, first_chunk, krow); break;
                        case 7: shift_and_store<7>(buf, dst_row, first_chunk, krow); break;
                        default: shift_and_store<8>(buf, dst_row, first_chunk, krow); break;
                        }
                    }
                    ptx::fence_proxy_async();          // generic-proxy stores -> visible to the tensor core's async proxy
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive(bfull_bar + 8u * bs);
                        ptx::mbar_arrive(lempty_bar + 8u * ls);
                    }
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
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace shiftws

// Column tiles per work item: the split of the column range that keeps all CTAs busy to the end (items a little under a
// whole number of rounds of the grid), with runs long enough to amortise the copy of the weights into tensor memory.
uint32_t shift_ws_chunk(uint32_t mtiles, uint32_t tiles_n, uint32_t num_sms) {
    uint32_t best = tiles_n;
    double best_eff = 0.0;
    for (uint32_t parts = 1; parts <= tiles_n; ++parts) {
        const uint32_t chunk = (tiles_n + parts - 1u) / parts;
        if (chunk < 8u && parts > 1u) break;
        const uint32_t chunks = (tiles_n + chunk - 1u) / chunk;
        const uint64_t items = (uint64_t)mtiles * chunks;
        const uint64_t rounds = (items + num_sms - 1u) / num_sms;
        // the busiest CTA runs `rounds` items of up to `chunk` tiles (+1 tile-equivalent per item for the weight copy)
        const double eff = (double)mtiles * tiles_n / ((double)rounds * (chunk + 1u) * num_sms);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = chunk; }
    }
    return best;
}

bool shift_ws_supported(const WaveArgs &a) {
    return a.gather_mode == GATHER_BOX && a.box_h >= 16u && kStageK % a.box_h == 0u && a.num_kstages <= (uint32_t)shiftws::kMaxKS && a.num_col_tiles64 % 2u == 0u &&
           (a.frame_len ? a.frame_len : a.pitch) % (uint32_t)shiftws::kN == 0u && a.k_splits == 1u && a.peers == nullptr;
}

cudaError_t launch_wave_umma_shift_ws(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s) {
    if (!shift_ws_supported(a) || d.n_tile != (uint32_t)shiftws::kN || d.ws_chunk == 0u) return cudaErrorInvalidValue;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    using KernelFn = void (*)(const CUtensorMap, const WaveArgs, const UmmaDesc);
    static const KernelFn fns[2] = {shiftws::k44_wave_umma_shift_ws_kernel<1>, shiftws::k44_wave_umma_shift_ws_kernel<2>};
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        for (KernelFn f : fns) {
            e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shiftws::kSmemBytes);
            if (e != cudaSuccess) return e;
        }
        attr_done[dev] = true;
    }
    const uint32_t mtiles = (a.cout + kTileM - 1) / kTileM;
    const uint32_t tiles_n = a.num_col_tiles64 / 2u;
    const uint32_t items = mtiles * ((tiles_n + d.ws_chunk - 1u) / d.ws_chunk);
    const uint32_t grid = items < (uint32_t)num_sms ? items : (uint32_t)num_sms;
    const uint32_t ag = d.ws_groups == 1u ? 1u : 2u;
    fns[ag - 1u]<<<grid, 32 * shiftws::kFirstAligner + 128 * ag, shiftws::kSmemBytes, s>>>(tmap, a, d);
    return cudaGetLastError();
}

}  // namespace k44b
