// The persistent streaming tcgen05 wave kernel (template) and its launch helpers. Instantiated per tile width in
// k44_stream_n64.cu / _n128.cu / _n256.cu so that the variants compile in parallel.
//
//   warp 0   producer: per 64-synapse stage one linear bulk copy of the packed weight block and one TMA box per run of
//            substrate rows (128-byte swizzle), completing on an mbarrier;
//   warp 1   a single thread issues tcgen05.mma (M=128 neurons, N=64..256 columns, K=16) with FP32 accumulators in tensor
//            memory, double-buffered across tiles;
//   warps 2-5 epilogue: tcgen05.ld -> bias -> activation -> residual -> FP16 RTE -> canvas rows.
// Replaces the roles of the reference's three mma.sync kernels and its tcgen05 prototype
// (kernels/cuda/kernel44_cuda_pack.cuh:242-286, 370-391, 438-623) for run-structured and scattered-row gathers.
// Every wait on a barrier is bounded in time; on expiry the kernel records a status bit, drains its own copies, frees its
// tensor memory and returns.
#pragma once
#include "k44_kernels.cuh"
#include "k44_epilogue.cuh"
#include "k44_ptx.cuh"

namespace k44b {

constexpr int kUmmaThreads = 192;

// STAGES_SEL == 0: deep pipeline, one CTA per SM (streaming waves with many tiles).
// STAGES_SEL == 1: 4 stages, two CTAs per SM (small waves: more CTAs in flight, split-K).
// MB: 128-neuron blocks per tile. 1: tiles of 128 neurons, two accumulators in tensor memory so that the epilogue of one
// tile overlaps the main loop of the next. 2 (256 columns only): tiles of 256 neurons — two blocks that share one gathered
// operand, each with its own weights and accumulator (all 512 tensor-memory columns, no second buffer): half the operand
// bytes per flop, for the tensor-bound regime of large neuron groups.
template <int N_TILE, int STAGES_SEL, int MB = 1>
struct UmmaCfg {
    static_assert(MB == 1 || (MB == 2 && N_TILE == 256 && STAGES_SEL == 0), "two neuron blocks per tile: 256-column streaming tiles only");
    static constexpr int kColBlocks = N_TILE / 64;                                    // 64-column blocks per tile
    static constexpr uint32_t kXBytes = (uint32_t)kColBlocks * kStageK * 128u;        // 8 KiB per 64 columns
    static constexpr uint32_t kWBytes = (uint32_t)MB * kStageWBytes;                  // weight blocks of a stage
    static constexpr uint32_t kStageBytes = kWBytes + kXBytes;
    static constexpr int kStages = MB == 2 ? 3 : (STAGES_SEL == 1 ? 4 : ((N_TILE == 64) ? 8 : (N_TILE == 128 ? 6 : 4)));
    static constexpr int kCtasPerSm = STAGES_SEL == 1 ? 2 : 1;
    static constexpr int kAccBufs = MB == 2 ? 1 : 2;                                  // accumulator buffers in tensor memory
    static constexpr uint32_t kTmemCols = 2u * N_TILE;
    // epilogue staging. One CTA per SM: two blocks of 128 rows x 128 bytes (one 64-column block of the output tile each, handed
    // to the copy engine in turn; the per-warp staging of the register-store path lives in the same space). Two CTAs per SM:
    // 128 rows x (64 + 16 pad) bytes for the register-store path only.
    static constexpr bool kTmaOut = STAGES_SEL == 0;
    static constexpr uint32_t kOutBlockBytes = 128u * 128u;
    static constexpr uint32_t kOutStageBytes = kTmaOut ? 2u * kOutBlockBytes : 128u * 80u;
    static constexpr uint32_t kSmemBytes = 1024u /*alignment slack*/ + (uint32_t)kStages * kStageBytes + kOutStageBytes + 256u;
};


// Work item = (neuron tile, column tile, K split). With splits == 1 the epilogue writes the canvas directly.
// With splits > 1 every item adds its partial accumulator into an FP32 scratch tile ([column][neuron] so that
// a warp's 32 neurons are contiguous), and the item that arrives last at the tile's counter applies the
// epilogue, stores the rows and leaves scratch and counter zeroed for the next launch. Nobody waits.
// ROWS_MODE != 0: the gather table holds one canvas row per synapse (scattered single rows, box_h == 1), the kind of table
// the reference's own benchmark draws.
//   1  (default) four extra warps fetch them with 16-byte asynchronous copies straight into the swizzled layout (one warp
//      instruction = one row piece of up to 512 contiguous bytes) and report completion on the stage's barrier, warp 0 only
//      streams the weights — the way the producer threads of the reference's tcgen05 kernel work
//      (kernels/cuda/kernel44_cuda_pack.cuh:481-491);
//   2  warp 0 fetches them with gather-mode tensor copies: one instruction brings four rows, each from its own canvas row,
//      64 columns wide, into four consecutive 128-byte rows of the swizzled operand stage; byte counting on the stage's
//      barrier as for boxes. Measured 3.4 times slower than mode 1 (the copy engine's cost is per 128-byte row piece); kept
//      for comparison (K44B_ROWS_MODE=2).
constexpr int kRowWarps = 4;
template <int N_TILE, int STAGES_SEL, int ROWS_MODE, int MB = 1>
__global__ void __launch_bounds__(kUmmaThreads + (ROWS_MODE == 1 ? 32 * kRowWarps : 0), UmmaCfg<N_TILE, STAGES_SEL, MB>::kCtasPerSm)
k44_wave_umma_kernel(const __grid_constant__ CUtensorMap tmap, const WaveArgs a, const UmmaDesc d) {
    using Cfg = UmmaCfg<N_TILE, STAGES_SEL, MB>;
    constexpr int STAGES = Cfg::kStages;
    constexpr bool ROWS = ROWS_MODE == 1;              // rows by asynchronous copies from their own warps
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows of 128 bytes
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_smem = smem_base;
    const uint32_t x_smem = smem_base + (uint32_t)STAGES * Cfg::kWBytes;
    const uint32_t out_smem = x_smem + (uint32_t)STAGES * Cfg::kXBytes;      // 1024-byte aligned (all stage sizes are multiples of 1024)
    const uint32_t ctl = out_smem + Cfg::kOutStageBytes;
    const uint32_t full_bar = ctl, empty_bar = ctl + 8u * STAGES;
    const uint32_t tfull_bar = ctl + 16u * STAGES, tempty_bar = tfull_bar + 16u;
    uint8_t *ctl_ptr = smem_raw + (ctl - ptx::smem_addr(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(ctl_ptr + 16 * STAGES + 32);
    volatile uint32_t *abort_word = tmem_slot + 1;
    volatile uint32_t *last_flag = tmem_slot + 2;
    volatile uint32_t *epi_ok = tmem_slot + 4;       // two slots, alternating per item
    volatile uint32_t *go_word = tmem_slot + 6;      // ROWS: set once the canvas may be read (peers' rows have arrived)
    uint8_t *out_stage = smem_raw + (out_smem - ptx::smem_addr(smem_raw));   // register-store path: 128 rows x 80 bytes, one 32-row block per epilogue warp

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tiles_n = a.num_col_tiles64 / Cfg::kColBlocks;
    const uint32_t mtiles = (a.cout + kTileM - 1) / kTileM;               // 128-neuron blocks of the wave
    const uint32_t mtiles_eff = (mtiles + (uint32_t)MB - 1u) / (uint32_t)MB; // tiles along the neurons
    const uint32_t splits = a.k_splits;
    const uint32_t total_items = mtiles_eff * tiles_n * splits;
    const uint32_t mtiles_per_group = a.mtiles_per_group;
    const uint32_t boxes_per_stage = kStageK / a.box_h;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar + 8u * s, ROWS ? 1u + 32u * kRowWarps : 1u);   // weights' byte count (+ one arrival per row-fetching thread)
            ptx::mbar_init(empty_bar + 8u * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar + 8u * b, 1);
            ptx::mbar_init(tempty_bar + 8u * b, 128);
        }
        *abort_word = 0;
        *go_word = a.peers ? 0u : 1u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_addr(const_cast<uint32_t *>(tmem_slot)), Cfg::kTmemCols);
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
    // item -> (tile, split) and the split's K-stage range
    auto decode = [&](uint32_t item, uint32_t &tile, uint32_t &ks0, uint32_t &ks1) {
        tile = item / splits;
        const uint32_t sp = item % splits;
        ks0 = sp * a.kstages_per_split;
        ks1 = min(a.num_kstages, ks0 + a.kstages_per_split);
    };

    // bytes a stage's barrier has to see: the tile's weight blocks (a last tile may hold a single block) and, unless the rows
    // come through ordinary asynchronous copies, the gathered rows
    auto stage_tx_bytes = [&](uint32_t nblk) -> uint32_t { return nblk * kStageWBytes + (ROWS ? 0u : Cfg::kXBytes); };

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) ptx::prefetch_tensormap(&tmap);
        const uint64_t pol_w = ptx::policy_evict_first();   // weights are streamed once
        const uint64_t pol_x = ptx::policy_evict_last();    // substrate rows are shared between groups
        // the weight blocks of K stage `ks` of the tile whose first block is `mt`, into pipeline slot `slot`
        auto issue_weights = [&](uint32_t slot, uint32_t mt, uint32_t nblk, uint32_t ks) {
            ptx::mbar_arrive_expect_tx(full_bar + 8u * slot, stage_tx_bytes(nblk));
            for (uint32_t b = 0; b < nblk; ++b)
                ptx::bulk_g2s(w_smem + slot * Cfg::kWBytes + b * kStageWBytes,
                              a.w_tiles + ((uint64_t)(mt + b) * a.num_kstages + ks) * (kStageWBytes / 16u), kStageWBytes, full_bar + 8u * slot, pol_w);
        };
        uint32_t issued = 0, pre = 0;
        bool ok = true;
        if (a.peers) {                       // neuron-sharded plan: the peers' rows of the previous launches must have arrived
            uint32_t okp = 1u;
            if (lane == 0) {
                // the weights never depend on a peer: the blocks of the first pipeline slots go out before the wait
                for (uint32_t item = blockIdx.x; item < total_items && pre < (uint32_t)STAGES; item += gridDim.x) {
                    uint32_t tile, ks0, ks1;
                    decode(item, tile, ks0, ks1);
                    const uint32_t mt = (tile / tiles_n) * (uint32_t)MB, nblk = min((uint32_t)MB, mtiles - mt);
                    for (uint32_t ks = ks0; ks < ks1 && pre < (uint32_t)STAGES; ++ks, ++pre) issue_weights(pre, mt, nblk, ks);
                }
                okp = peer_wait_ready(a.peers, d.wait_cycles, a.peer_slack) ? 1u : 0u;
                asm volatile("fence.proxy.async.global;" ::: "memory");   // rows written by peers' plain stores -> this thread's tensor copies
                if (!okp) { atomicOr(a.status, (uint32_t)ST_TIMEOUT_PEER); *abort_word = 1u; }
                else { __threadfence_block(); *go_word = 1u; }
            }
            ok = __shfl_sync(0xffffffffu, okp, 0) != 0u;
            pre = __shfl_sync(0xffffffffu, pre, 0);
        }
        for (uint32_t item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            uint32_t tile, ks0, ks1;
            decode(item, tile, ks0, ks1);
            const uint32_t mt = (tile / tiles_n) * (uint32_t)MB, ct = tile % tiles_n, nblk = min((uint32_t)MB, mtiles - mt);
            const uint32_t *rows = a.gather + (uint64_t)(mt / mtiles_per_group) * a.boxes_per_group;
            uint32_t cached = 0, cached_base = 0xffffffffu;
            for (uint32_t ks = ks0; ks < ks1 && ok; ++ks) {
                const uint32_t stage = issued % STAGES, ph = (issued / STAGES) & 1u;
                if (lane == 0 && issued >= pre) {
                    ok = wait(empty_bar + 8u * stage, ph ^ 1u);
                    if (ok) issue_weights(stage, mt, nblk, ks);   // weights first: they do not need the run table
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                // One TMA box per (run, 64-column block). The whole warp fetches 32 table entries at a time (an entry is
                // row | token shift << 28; the shift is only used by other kernels). Issuing a tensor copy costs its thread
                // of the order of a hundred cycles, so when a step has several boxes they go out from different lanes in one
                // warp instruction; a step with a single box (runs of 64 rows, 64-column tiles) is issued by lane 0 as before.
                const uint32_t per_stage = boxes_per_stage * (uint32_t)Cfg::kColBlocks;     // at most 8 x 4
                if (ROWS_MODE == 2) {
                    // 16 row quads x column blocks per stage: copy q = lane, lane + 32, ... takes quad q / blocks of block q % blocks
                    constexpr uint32_t kCopies = 16u * (uint32_t)Cfg::kColBlocks;
                    const uint4 *quads = reinterpret_cast<const uint4 *>(rows + (uint64_t)ks * kStageK);
#pragma unroll
                    for (uint32_t q = lane; q < kCopies; q += 32u) {
                        const uint32_t r4 = q / (uint32_t)Cfg::kColBlocks, cb = q % (uint32_t)Cfg::kColBlocks;
                        const uint4 e = __ldg(quads + r4);
                        ptx::tma_gather4_2d(x_smem + stage * Cfg::kXBytes + cb * (kStageK * 128u) + r4 * 512u, &tmap, (int32_t)(ct * N_TILE + cb * 64u),
                                            (int32_t)(e.x & kBoxRowMask), (int32_t)(e.y & kBoxRowMask), (int32_t)(e.z & kBoxRowMask),
                                            (int32_t)(e.w & kBoxRowMask), full_bar + 8u * stage, pol_x);
                    }
                } else if (!ROWS) {
                    const uint32_t bi0 = ks * boxes_per_stage;
                    if ((bi0 & ~31u) != cached_base) {       // the boxes of one step never straddle a group of 32 entries
                        cached_base = bi0 & ~31u;
                        cached = (cached_base + lane < a.boxes_per_group) ? __ldg(rows + cached_base + lane) : 0u;
                    }
                    const uint32_t b = lane / (uint32_t)Cfg::kColBlocks, cb = lane % (uint32_t)Cfg::kColBlocks;
                    const uint32_t row = __shfl_sync(0xffffffffu, cached, (bi0 + b) & 31u) & kBoxRowMask;
                    if (lane < per_stage)
                        ptx::tma_load_2d(x_smem + stage * Cfg::kXBytes + cb * (kStageK * 128u) + b * a.box_h * 128u, &tmap,
                                         (int32_t)(ct * N_TILE + cb * 64u), (int32_t)row, full_bar + 8u * stage, pol_x);
                }
                ++issued;
            }
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
            *abort_word = 1u;
            // wait (bounded) for copies already in flight before this CTA's shared memory goes away; slots whose weights went out
            // ahead of the peer wait but whose rows never followed get the missing bytes taken off their count first
            if (!ROWS) for (uint32_t i = issued; i < pre; ++i) ptx::mbar_complete_tx(full_bar + 8u * i, Cfg::kXBytes);
            const uint32_t last = issued > pre ? issued : pre;
            const uint32_t first = last > (uint32_t)STAGES ? last - STAGES : 0u;
            for (uint32_t i = first; i < last; ++i) {
                const long long t0 = clock64();
                bool done = false;
                while (!done && (unsigned long long)(clock64() - t0) < d.wait_cycles)
                    done = ptx::mbar_try_wait(full_bar + 8u * (i % STAGES), (i / STAGES) & 1u);
                if (!done) atomicOr(a.status, (uint32_t)ST_TIMEOUT_DRAIN);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t consumed = 0, iter = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++iter) {
                uint32_t tile, ks0, ks1;
                decode(item, tile, ks0, ks1);
                const uint32_t nblk = min((uint32_t)MB, mtiles - (tile / tiles_n) * (uint32_t)MB);
                const uint32_t acc = iter % (uint32_t)Cfg::kAccBufs;
                ok = wait(tempty_bar + 8u * acc, ((iter / (uint32_t)Cfg::kAccBufs) & 1u) ^ 1u);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * N_TILE;
                for (uint32_t ks = ks0; ks < ks1; ++ks) {
                    const uint32_t stage = consumed % STAGES, ph = (consumed / STAGES) & 1u;
                    ok = wait(full_bar + 8u * stage, ph) && *abort_word == 0u;   // (a producer that gave up completes its barriers itself)
                    if (!ok) break;
                    ptx::tc_fence_after();
                    if (ROWS) ptx::fence_proxy_async();      // rows arrived through ordinary asynchronous copies: order them before the tensor core's reads
                    const uint64_t a0 = d.a_base | (uint64_t)(((w_smem + stage * Cfg::kWBytes) >> 4) & 0x3fffu);
                    const uint64_t b0 = d.b_base | (uint64_t)(((x_smem + stage * Cfg::kXBytes) >> 4) & 0x3fffu);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kStageK / 16u; ++k4) {
                        ptx::umma_f16(d_tmem, a0 + (uint64_t)(k4 * d.a_k_step), b0 + (uint64_t)(k4 * d.b_k_step), d.idesc,
                                      (ks != ks0 || k4 != 0u) ? 1u : 0u);
                        if (MB == 2 && nblk == 2u)       // second neuron block: its own weights and accumulator columns, the same operand
                            ptx::umma_f16(d_tmem + (uint32_t)N_TILE, a0 + (uint64_t)(kStageWBytes >> 4) + (uint64_t)(k4 * d.a_k_step),
                                          b0 + (uint64_t)(k4 * d.b_k_step), d.idesc, (ks != ks0 || k4 != 0u) ? 1u : 0u);
                    }
                    ptx::umma_commit(empty_bar + 8u * stage);      // stage reusable once these MMAs retire
                    ++consumed;
                }
                if (ok) ptx::umma_commit(tfull_bar + 8u * acc);     // accumulator complete
            }
            if (!ok) {
                if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_MMA);
                *abort_word = 1u;
            }
        }
        __syncwarp();
    } else if (ROWS && warp >= 6u) {
        // ---------------- row fetchers (scattered single rows) ----------------
        // warp w of the four takes rows 16w .. 16w+15 of every 64-synapse stage; one instruction copies one row's N_TILE
        // columns (lane l: 16-byte chunk l, and l + 32 .. for tiles wider than 256 columns there is no such tile)
        const uint32_t rw = warp - 6u;
        constexpr uint32_t kChunksPerRow = (uint32_t)N_TILE / 8u;                     // 8, 16 or 32 chunks of 16 bytes
        constexpr uint32_t kRowsPerInstr = 32u / kChunksPerRow;                      // 4, 2 or 1 rows per warp instruction
        const uint32_t sub_row = lane / kChunksPerRow, chunk = lane % kChunksPerRow;
        const uint32_t cb = chunk >> 3, cc = chunk & 7u;
        bool ok = true;
        {   // the canvas may be read once the peers' rows are in (no peers: at once)
            uint32_t okw = 1u;
            if (lane == 0) {
                const long long t0 = clock64();
                while (*go_word == 0u) {
                    if (*abort_word != 0u || (unsigned long long)(clock64() - t0) > d.wait_cycles) { okw = 0u; break; }
                }
                __threadfence_system();
            }
            ok = __shfl_sync(0xffffffffu, okw, 0) != 0u;
        }
        // The stages this CTA will work through, as a cursor: (item, K stage) -> this warp's 16 table entries and the tile's first
        // column. (Asking L2 for the rows a dozen stages ahead — bulk prefetches or per-line prefetch instructions — was measured
        // and brought nothing: the row fetch is bound on the SM side, not by the latency of the 80 M-row substrate.)
        struct Cursor { uint32_t item, ks, ks1; const uint32_t *rows; const __half *col; bool valid; };
        auto seek = [&](Cursor &c, uint32_t item) {
            c.item = item;
            c.valid = item < total_items;
            if (!c.valid) return;
            uint32_t tile, ks0;
            decode(item, tile, ks0, c.ks1);
            c.ks = ks0;
            const uint32_t mt = (tile / tiles_n) * (uint32_t)MB, ct = tile % tiles_n;
            c.rows = a.gather + (uint64_t)(mt / mtiles_per_group) * a.boxes_per_group + 16u * rw;
            c.col = a.canvas + (uint64_t)ct * N_TILE;
            if (c.ks >= c.ks1) c.valid = false;
        };
        auto step = [&](Cursor &c) { if (++c.ks >= c.ks1) seek(c, c.item + gridDim.x); };
        Cursor f;
        seek(f, blockIdx.x);
        // this warp's 16 table entries travel one stage ahead of their use, so that their latency hides behind the previous
        // stage's copies instead of standing in front of every stage
        uint32_t nxt = (f.valid && lane < 16u) ? __ldg(f.rows + (uint64_t)f.ks * kStageK + lane) : 0u;
        uint32_t issued = 0;
        while (f.valid && ok) {
            const uint32_t stage = issued % STAGES, ph = (issued / STAGES) & 1u;
            const uint32_t cur = nxt;                                                                     // this warp's 16 rows of the stage
            {
                Cursor g = f;
                step(g);
                nxt = (g.valid && lane < 16u) ? __ldg(g.rows + (uint64_t)g.ks * kStageK + lane) : 0u;
            }
            uint32_t okw = 1u;
            if (lane == 0) okw = wait(empty_bar + 8u * stage, ph ^ 1u) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, okw, 0) != 0u;
            if (!ok) break;
            const uint32_t dst0 = x_smem + stage * Cfg::kXBytes + cb * (kStageK * 128u);
            const __half *col0 = f.col + chunk * 8u;
#pragma unroll
            for (uint32_t i = 0; i < 16u / kRowsPerInstr; ++i) {
                const uint32_t rl = i * kRowsPerInstr + sub_row;                  // row inside this warp's 16
                const uint32_t row = __shfl_sync(0xffffffffu, cur, rl) & kBoxRowMask;
                const uint32_t k = 16u * rw + rl;                                 // row inside the stage
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + k * 128u + ((cc ^ (k & 7u)) << 4)),
                             "l"(col0 + (uint64_t)row * a.pitch)
                             : "memory");
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full_bar + 8u * stage) : "memory");
            step(f);
            ++issued;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");     // nothing of this thread is in flight when the CTA's shared memory goes away
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
            *abort_word = 1u;
        }
    } else {
        // ---------------- epilogue ----------------
        const uint32_t quarter = warp & 3u;                  // TMEM lanes this warp may read
        const bool has_map = a.cout_map != nullptr;
        const bool tma_out = a.out_maps != nullptr && !has_map && splits == 1u;
        uint32_t blocks_out = 0;                             // 64-column blocks handed to the copy engine so far
        uint32_t iter = 0;
        bool ok = true;
        for (uint32_t item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++iter) {
            uint32_t tile, ks0, ks1;
            decode(item, tile, ks0, ks1);
            const uint32_t mt = (tile / tiles_n) * (uint32_t)MB, ct = tile % tiles_n, acc = iter % (uint32_t)Cfg::kAccBufs;
            const uint32_t nblk = min((uint32_t)MB, mtiles - mt);
            // one thread waits (bounded) and tells the other 127, so that all four warps take the same branch
            if (threadIdx.x == 64u) epi_ok[iter & 1u] = (wait(tfull_bar + 8u * acc, (iter / (uint32_t)Cfg::kAccBufs) & 1u) && *abort_word == 0u) ? 1u : 0u;
            epilogue_bar_sync();
            ok = epi_ok[iter & 1u] != 0u;
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t r_in_tile = quarter * 32u + lane;
            const uint32_t j = mt * kTileM + r_in_tile;
            const bool live = j < a.cout;
            const uint32_t oj = (live && has_map) ? a.cout_map[j] : j;
            const float bias = (live && a.bias) ? __half2float(a.bias[j]) : 0.0f;
            const uint64_t o = (uint64_t)oj * a.pitch + (uint64_t)ct * N_TILE;
            if (Cfg::kTmaOut && (tma_out || MB == 2)) {
                // per 128-neuron block and 64-column block: wait until the copy that last read this staging block is done with it,
                // convert and park the block, hand it to the copy engine (own canvas and peers)
#pragma unroll 1
                for (uint32_t nb = 0; nb < nblk; ++nb) {
                    const uint32_t jb = j + nb * kTileM;
                    const bool live_b = jb < a.cout;
                    const float bias_b = nb == 0u ? bias : ((live_b && a.bias) ? __half2float(a.bias[jb]) : 0.0f);
#pragma unroll 1
                    for (uint32_t cb = 0; cb < (uint32_t)Cfg::kColBlocks; ++cb, ++blocks_out) {
                        const uint32_t block_smem = out_smem + (blocks_out & 1u) * Cfg::kOutBlockBytes;
                        if (threadIdx.x == 64u) ptx::bulk_wait_group_read<1>();
                        epilogue_bar_sync();
#pragma unroll 1
                        for (uint32_t half = 0; half < 2u; ++half) {
                            uint32_t v[32];
                            ptx::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + (MB == 2 ? nb : acc) * N_TILE + cb * 64u + half * 32u, v);
                            ptx::tmem_ld_wait();
                            float f[32];
#pragma unroll
                            for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(v[e]);
                            stage_half_block(a, f, bias_b, live_b, jb, (uint64_t)ct * N_TILE + cb * 64u + half * 32u, block_smem, r_in_tile, half);
                        }
                        if (nb + 1u == nblk && cb + 1u == (uint32_t)Cfg::kColBlocks) {      // accumulators read out: the next item's MMAs may start
                            ptx::tc_fence_before();
                            ptx::mbar_arrive(tempty_bar + 8u * acc);
                        }
                        ptx::fence_proxy_async();                        // this thread's shared-memory stores -> visible to the copy engine
                        epilogue_bar_sync();
                        if (threadIdx.x == 64u) {
                            const int32_t x = (int32_t)(ct * (uint32_t)N_TILE + cb * 64u), y = (int32_t)((mt + nb) * kTileM);
                            for (uint32_t m = 0; m < a.n_out_maps; ++m) ptx::tma_store_2d(a.out_maps + m, x, y, block_smem);
                            ptx::bulk_commit_group();
                        }
                    }
                }
            } else if (splits == 1u) {
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
            } else {
                float *sc = a.scratch + (uint64_t)tile * (N_TILE * kTileM) + r_in_tile;
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < (uint32_t)N_TILE; c0 += 32u) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * N_TILE + c0, v);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) atomicAdd(sc + (uint64_t)(c0 + e) * kTileM, __uint_as_float(v[e]));
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(tempty_bar + 8u * acc);      // accumulator free: the next item's MMAs may start
                __threadfence();
                epilogue_bar_sync();
                if (threadIdx.x == 64u) {
                    const uint32_t prev = atomicAdd(a.counters + tile, 1u);
                    *last_flag = (prev == splits - 1u) ? 1u : 0u;
                }
                epilogue_bar_sync();
                if (*last_flag != 0u) {
                    __threadfence();
#pragma unroll 1
                    for (uint32_t c0 = 0; c0 < (uint32_t)N_TILE; c0 += 32u) {
                        float f[32];
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            float *p = sc + (uint64_t)(c0 + e) * kTileM;
                            f[e] = __ldcg(p);
                            __stcg(p, 0.0f);
                        }
                        stage_and_store(a, f, bias, has_map, live, oj, (uint64_t)ct * N_TILE + c0, out_stage + quarter * (32u * 80u), lane);
                    }
                    if (threadIdx.x == 64u) a.counters[tile] = 0u;
                }
                epilogue_bar_sync();                          // last_flag is rewritten by the next item
            }
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_EPILOGUE);
            *abort_word = 1u;
        }
        if (Cfg::kTmaOut && (tma_out || MB == 2) && threadIdx.x == 64u) {
            ptx::bulk_wait_group<0>();       // the tile copies have been written (and no longer read this CTA's shared memory)
            ptx::fence_proxy_async_global(); // ... and are ordered before this thread's generic-proxy fence and counter below
        }
        if (a.peers) {                       // this CTA's rows are stored here and on every peer: count it as done
            epilogue_bar_sync();             // the storing threads' writes are ordered before the one fence below (cumulativity)
            if (threadIdx.x == 64u) peer_signal_done(a.peers, gridDim.x);
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <int N_TILE, int SEL, int ROWS = 0, int MB = 1>
static cudaError_t umma_attr() {
    return cudaFuncSetAttribute(k44_wave_umma_kernel<N_TILE, SEL, ROWS, MB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)UmmaCfg<N_TILE, SEL, MB>::kSmemBytes);
}


template <int N_TILE, int SEL, int ROWS = 0, int MB = 1>
static cudaError_t umma_launch(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s) {
    using Cfg = UmmaCfg<N_TILE, SEL, MB>;
    const uint32_t mtiles = ((a.cout + kTileM - 1) / kTileM + (uint32_t)MB - 1u) / (uint32_t)MB;
    const uint32_t items = mtiles * (a.num_col_tiles64 / (N_TILE / 64u)) * a.k_splits;
    const uint32_t cap = (uint32_t)num_sms * Cfg::kCtasPerSm;
    const uint32_t grid = items < cap ? items : cap;
    if (MB == 2 && (a.k_splits != 1u || !a.out_maps || a.cout_map || (a.mtiles_per_group & 1u))) return cudaErrorInvalidValue;
    k44_wave_umma_kernel<N_TILE, SEL, ROWS, MB><<<grid, kUmmaThreads + (ROWS == 1 ? 32 * kRowWarps : 0), Cfg::kSmemBytes, s>>>(tmap, a, d);
    return cudaGetLastError();
}

}  // namespace k44b
