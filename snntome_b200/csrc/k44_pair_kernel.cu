// Streaming tcgen05 wave kernel on CTA pairs (cta_group::2), for the tensor-bound regime of large neuron groups.
//
// A tile is 256 neurons x 256 columns and belongs to a pair of CTAs (a cluster of two, on two SMs). CTA r of the pair
// holds the weights of neurons 128r .. 128r+127 and the gathered operand of columns 128r .. 128r+127; one thread of CTA 0
// issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16), which reads both CTAs' shared memory and leaves each CTA its
// own 128 neurons x 256 columns in its own tensor memory. Against the one-CTA kernel (128 x 256 tiles) every flop needs a
// third less operand traffic through L2 and, above all, a third less shared-memory read bandwidth, which is what bounds
// the one-CTA kernel near two thirds of the tensor rate (per 128-cycle MMA it reads 4 KiB of weights and 8 KiB of operand
// while the copies write as much again; a pair reads 4 + 4 KiB per SM).
//
//   warp 0   producer of its CTA: per 64-synapse stage one tensor copy of its weight block (16 KiB; the packed weights seen as
//            rows of 128 bytes) and, for run tables, one TMA box per run and 64-column block of its half of the columns;
//            both CTAs' copies count their bytes on the stage's barrier in CTA 0 (pair-scoped copies, no multicast);
//   warp 1   CTA 0: one thread issues the pair's MMAs and commits to the barriers of both CTAs; CTA 1: allocates and frees,
//            and with scattered rows forwards the completion of its row copies to CTA 0;
//   warps 2-5 epilogue of the CTA's own 128 neurons out of double-buffered tensor memory: tile copies (k44_epilogue.cuh);
//   warps 6-9 (scattered single rows only) fetch the CTA's half of every row with 16-byte asynchronous copies.
// This is the role of the reference's own Blackwell kernel (kernels/cuda/kernel44_cuda_pack.cuh:438-623: 256 x 256 tiles on
// one CTA, cta_group::1); the fused epilogue, the chained layout and the pairing are this build's.
// Every wait is bounded; on expiry the kernel records a status bit and both CTAs leave through the common exit, where
// the pair meets once more before its tensor memory is freed.
#include "k44_kernels.cuh"
#include "k44_epilogue.cuh"
#include "k44_ptx.cuh"

namespace k44b {
namespace pairwave {

constexpr uint32_t kTileN = 256;                                   // columns per pair tile
constexpr uint32_t kHalfN = 128;                                   // columns one CTA stages
constexpr uint32_t kXBytes = (kHalfN / 64u) * kStageK * 128u;      // 16 KiB: two 64-column blocks of 64 rows
constexpr uint32_t kStageBytes = kStageWBytes + kXBytes;           // 32 KiB
constexpr int kStages = 6;
constexpr uint32_t kOutBlockBytes = 128u * 128u;
constexpr uint32_t kSmemBytes = 1024u + (uint32_t)kStages * kStageBytes + 2u * kOutBlockBytes + 256u;
constexpr uint32_t kTmemCols = 512;                                // two accumulators of 256 columns
constexpr int kRowWarps = 4;
constexpr int kThreads = 192;

template <int ROWS>   // 0: run table (TMA boxes), 1: one row per synapse (asynchronous 16-byte copies from four extra warps)
__global__ void __launch_bounds__(kThreads + (ROWS ? 32 * kRowWarps : 0), 1)
k44_wave_umma_pair_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap wmap, const WaveArgs a, const UmmaDesc d) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_smem = smem_base;
    const uint32_t x_smem = smem_base + (uint32_t)kStages * kStageWBytes;
    const uint32_t out_smem = x_smem + (uint32_t)kStages * kXBytes;
    const uint32_t ctl = out_smem + 2u * kOutBlockBytes;
    const uint32_t full_bar = ctl, empty_bar = ctl + 8u * kStages;             // full: used in CTA 0 only; empty: in both
    const uint32_t tfull_bar = ctl + 16u * kStages, tempty_bar = tfull_bar + 16u;   // tfull: both; tempty: CTA 0 only
    const uint32_t xdone_bar = tempty_bar + 16u;                                // CTA 1, scattered rows: its own copies of a stage landed (kStages of them)
    uint8_t *ctl_ptr = smem_raw + (ctl - ptx::smem_addr(smem_raw));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(ctl_ptr + 16 * kStages + 32 + 8 * kStages);
    volatile uint32_t *abort_word = tmem_slot + 1;
    volatile uint32_t *epi_ok = tmem_slot + 2;      // two slots

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = ptx::cluster_ctarank();                               // 0: issues the MMAs
    const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const uint32_t tiles_n = a.num_col_tiles64 / 4u;
    const uint32_t mpairs = ((a.cout + kTileM - 1) / kTileM) / 2u;              // the host guarantees an even block count
    const uint32_t total_items = mpairs * tiles_n;
    const uint32_t KS = a.num_kstages;
    const uint32_t boxes_per_stage = kStageK / a.box_h;
    const uint32_t lead_full = ptx::map_to_cta(full_bar, 0u);                   // the stage barriers of CTA 0, as seen from either CTA
    const uint32_t lead_tempty = ptx::map_to_cta(tempty_bar, 0u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            // bytes of both CTAs' tensor copies + CTA 0's announcement; scattered rows: + CTA 0's 128 row-fetching threads + one
            // forwarded arrival from CTA 1
            ptx::mbar_init(full_bar + 8u * s, ROWS ? 1u + 32u * kRowWarps + 1u : 1u);
            ptx::mbar_init(empty_bar + 8u * s, 1);
            ptx::mbar_init(xdone_bar + 8u * s, 32u * kRowWarps);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(tfull_bar + 8u * b, 1);
            ptx::mbar_init(tempty_bar + 8u * b, 256);                            // the epilogue threads of both CTAs
        }
        *abort_word = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_addr(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_arrive();                     // both CTAs' barriers exist before either signals the other
    ptx::cluster_wait();
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
    const uint32_t my_items = pair < total_items ? (total_items - pair + num_pairs - 1) / num_pairs : 0u;
    auto decode = [&](uint32_t it, uint32_t &mp, uint32_t &ct) { const uint32_t item = pair + it * num_pairs; mp = item / tiles_n; ct = item % tiles_n; };

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) { ptx::prefetch_tensormap(&tmap); ptx::prefetch_tensormap(&wmap); }
        const uint64_t pol_w = ptx::policy_evict_first();
        const uint64_t pol_x = ptx::policy_evict_last();
        uint32_t issued = 0;
        bool ok = true;
        for (uint32_t it = 0; it < my_items && ok; ++it) {
            uint32_t mp, ct;
            decode(it, mp, ct);
            const uint32_t mt = 2u * mp + rank;                                  // this CTA's 128-neuron block
            const uint32_t *rows = a.gather + (uint64_t)((2u * mp) / a.mtiles_per_group) * a.boxes_per_group;
            uint32_t cached = 0, cached_base = 0xffffffffu;
            for (uint32_t ks = 0; ks < KS && ok; ++ks, ++issued) {
                const uint32_t stage = issued % kStages, ph = (issued / kStages) & 1u;
                if (lane == 0) {
                    ok = wait(empty_bar + 8u * stage, ph ^ 1u);
                    if (ok) {
                        // CTA 0 announces the bytes of the whole pair; CTA 1's copies only deliver theirs
                        if (rank == 0u) ptx::mbar_arrive_expect_tx(full_bar + 8u * stage, 2u * kStageWBytes + (ROWS ? 0u : 2u * kXBytes));
                        ptx::tma_load_2d_pair(w_smem + stage * kStageWBytes, &wmap, 0, (int32_t)((mt * KS + ks) * kTileM), lead_full + 8u * stage, pol_w);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                if (!ROWS) {
                    // one box per (run, 64-column block of this CTA's half): lane l takes box l / 2 of block l % 2
                    const uint32_t bi0 = ks * boxes_per_stage;
                    if ((bi0 & ~31u) != cached_base) {
                        cached_base = bi0 & ~31u;
                        cached = (cached_base + lane < a.boxes_per_group) ? __ldg(rows + cached_base + lane) : 0u;
                    }
                    const uint32_t b = lane >> 1, cb = lane & 1u;
                    const uint32_t row = __shfl_sync(0xffffffffu, cached, (bi0 + b) & 31u) & kBoxRowMask;
                    if (lane < 2u * boxes_per_stage)
                        ptx::tma_load_2d_pair(x_smem + stage * kXBytes + cb * (kStageK * 128u) + b * a.box_h * 128u, &tmap,
                                              (int32_t)(ct * kTileN + rank * kHalfN + cb * 64u), (int32_t)row, lead_full + 8u * stage, pol_x);
                }
            }
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
            *abort_word = 1u;
        }
        // (copies in flight are drained at the common exit: CTA 0 waits for the stage barriers there)
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (CTA 0) ----------------
        if (lane == 0 && rank == 0u) {
            uint32_t consumed = 0;
            bool ok = true;
            for (uint32_t it = 0; it < my_items && ok; ++it) {
                const uint32_t acc = it & 1u;
                ok = wait(tempty_bar + 8u * acc, ((it >> 1) & 1u) ^ 1u);         // both CTAs' epilogues are done with this accumulator
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kTileN;
                for (uint32_t ks = 0; ks < KS; ++ks, ++consumed) {
                    const uint32_t stage = consumed % kStages, ph = (consumed / kStages) & 1u;
                    ok = wait(full_bar + 8u * stage, ph) && *abort_word == 0u;
                    if (!ok) break;
                    ptx::tc_fence_after();
                    if (ROWS) ptx::fence_proxy_async();
                    const uint64_t a0 = d.a_base | (uint64_t)(((w_smem + stage * kStageWBytes) >> 4) & 0x3fffu);
                    const uint64_t b0 = d.b_base | (uint64_t)(((x_smem + stage * kXBytes) >> 4) & 0x3fffu);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kStageK / 16u; ++k4)
                        ptx::umma_f16_pair(d_tmem, a0 + (uint64_t)(k4 * d.a_k_step), b0 + (uint64_t)(k4 * d.b_k_step), d.idesc, (ks != 0u || k4 != 0u) ? 1u : 0u);
                    ptx::umma_commit_pair(empty_bar + 8u * stage, 3);            // the stage is free again in both CTAs
                }
                if (ok) ptx::umma_commit_pair(tfull_bar + 8u * acc, 3);          // both CTAs' halves of the accumulator are complete
            }
            if (!ok) {
                if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_MMA);
                *abort_word = 1u;
            }
        } else if (ROWS && lane == 0) {
            // CTA 1, scattered rows: pass every completed stage of this CTA's row copies on to the stage barrier in CTA 0
            bool ok = true;
            uint32_t fwd = 0;
            for (uint32_t it = 0; it < my_items && ok; ++it)
                for (uint32_t ks = 0; ks < KS && ok; ++ks, ++fwd) {
                    const uint32_t stage = fwd % kStages, ph = (fwd / kStages) & 1u;
                    ok = wait(xdone_bar + 8u * stage, ph);
                    if (ok) { ptx::fence_proxy_async(); ptx::mbar_arrive_cluster(lead_full + 8u * stage); }
                }
            if (!ok) {
                if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
                *abort_word = 1u;
            }
        }
        __syncwarp();
    } else if (ROWS && warp >= 6u) {
        // ---------------- row fetchers: this CTA's 128 columns of every scattered row ----------------
        const uint32_t rw = warp - 6u;
        constexpr uint32_t kChunksPerRow = kHalfN / 8u;                          // 16 chunks of 16 bytes
        constexpr uint32_t kRowsPerInstr = 32u / kChunksPerRow;                  // 2 rows per warp instruction
        const uint32_t sub_row = lane / kChunksPerRow, chunk = lane % kChunksPerRow;
        const uint32_t cb = chunk >> 3, cc = chunk & 7u;
        uint32_t issued = 0;
        bool ok = true;
        for (uint32_t it = 0; it < my_items && ok; ++it) {
            uint32_t mp, ct;
            decode(it, mp, ct);
            const uint32_t *rows = a.gather + (uint64_t)((2u * mp) / a.mtiles_per_group) * a.boxes_per_group + 16u * rw;
            const __half *col0 = a.canvas + (uint64_t)ct * kTileN + rank * kHalfN + chunk * 8u;
            uint32_t nxt = (KS && lane < 16u) ? __ldg(rows + lane) : 0u;          // table entries travel one stage ahead of their use
            for (uint32_t ks = 0; ks < KS && ok; ++ks, ++issued) {
                const uint32_t stage = issued % kStages, ph = (issued / kStages) & 1u;
                const uint32_t cur = nxt;
                if (ks + 1u < KS && lane < 16u) nxt = __ldg(rows + (uint64_t)(ks + 1u) * kStageK + lane);
                uint32_t okw = 1u;
                if (lane == 0) okw = wait(empty_bar + 8u * stage, ph ^ 1u) ? 1u : 0u;
                ok = __shfl_sync(0xffffffffu, okw, 0) != 0u;
                if (!ok) break;
                const uint32_t dst0 = x_smem + stage * kXBytes + cb * (kStageK * 128u);
#pragma unroll
                for (uint32_t i = 0; i < 16u / kRowsPerInstr; ++i) {
                    const uint32_t rl = i * kRowsPerInstr + sub_row;
                    const uint32_t row = __shfl_sync(0xffffffffu, cur, rl) & kBoxRowMask;
                    const uint32_t k = 16u * rw + rl;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + k * 128u + ((cc ^ (k & 7u)) << 4)),
                                 "l"(col0 + (uint64_t)row * a.pitch)
                                 : "memory");
                }
                // CTA 0's threads arrive on the stage barrier themselves; CTA 1's arrive on a barrier of their own, and one of
                // them passes the completed stage on to CTA 0 (an arrival cannot be bound to another CTA's barrier directly)
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"((rank == 0u ? full_bar : xdone_bar) + 8u * stage) : "memory");
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PRODUCER);
            *abort_word = 1u;
        }
    } else if (warp >= 2u && warp < 6u) {
        // ---------------- epilogue: this CTA's 128 neurons x 256 columns ----------------
        const uint32_t quarter = warp & 3u;
        uint32_t blocks_out = 0;
        bool ok = true;
        for (uint32_t it = 0; it < my_items && ok; ++it) {
            uint32_t mp, ct;
            decode(it, mp, ct);
            const uint32_t mt = 2u * mp + rank, acc = it & 1u;
            if (threadIdx.x == 64u) epi_ok[it & 1u] = (wait(tfull_bar + 8u * acc, (it >> 1) & 1u) && *abort_word == 0u) ? 1u : 0u;
            epilogue_bar_sync();
            ok = epi_ok[it & 1u] != 0u;
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t r_in_tile = quarter * 32u + lane;
            const uint32_t j = mt * kTileM + r_in_tile;
            const bool live = j < a.cout;
            const float bias = (live && a.bias) ? __half2float(a.bias[j]) : 0.0f;
#pragma unroll 1
            for (uint32_t cb = 0; cb < kTileN / 64u; ++cb, ++blocks_out) {
                const uint32_t block_smem = out_smem + (blocks_out & 1u) * kOutBlockBytes;
                if (threadIdx.x == 64u) ptx::bulk_wait_group_read<1>();
                epilogue_bar_sync();
#pragma unroll 1
                for (uint32_t half = 0; half < 2u; ++half) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * kTileN + cb * 64u + half * 32u, v);
                    ptx::tmem_ld_wait();
                    float f[32];
#pragma unroll
                    for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(v[e]);
                    stage_half_block(a, f, bias, live, j, (uint64_t)ct * kTileN + cb * 64u + half * 32u, block_smem, r_in_tile, half);
                }
                if (cb + 1u == kTileN / 64u) {                                   // accumulator read out: tell the issuing CTA
                    ptx::tc_fence_before();
                    ptx::mbar_arrive_cluster(lead_tempty + 8u * acc);
                }
                ptx::fence_proxy_async();
                epilogue_bar_sync();
                if (threadIdx.x == 64u) {
                    const int32_t x = (int32_t)(ct * kTileN + cb * 64u), y = (int32_t)(mt * kTileM);
                    for (uint32_t m = 0; m < a.n_out_maps; ++m) ptx::tma_store_2d(a.out_maps + m, x, y, block_smem);
                    ptx::bulk_commit_group();
                }
            }
        }
        if (!ok && lane == 0) {
            if (*abort_word == 0u) atomicOr(a.status, (uint32_t)ST_TIMEOUT_EPILOGUE);
            *abort_word = 1u;
        }
        if (threadIdx.x == 64u) ptx::bulk_wait_group<0>();   // the tile copies no longer read this CTA's shared memory
    }
    // ---------------- common exit ----------------
    // Every copy this CTA issued counts on a stage barrier of CTA 0 and is consumed by the MMA issuer there in the normal
    // course; after an abort CTA 0 waits (bounded) for the stages still in flight so that no copy lands in shared memory
    // that has been given back. Then the pair meets: neither CTA frees tensor memory or leaves while the other may still
    // signal its barriers or write its accumulators.
    ptx::tc_fence_before();
    __syncthreads();
    if (*abort_word != 0u && threadIdx.x == 0) {
        const long long t0 = clock64();
        while ((unsigned long long)(clock64() - t0) < 2000000ull) { }           // about a millisecond: copies in flight land
    }
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

template <int ROWS>
static cudaError_t launch(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, const CUtensorMap &wmap, int num_sms, cudaStream_t s) {
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        e = cudaFuncSetAttribute(k44_wave_umma_pair_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const uint32_t mpairs = ((a.cout + kTileM - 1) / kTileM) / 2u;
    const uint32_t items = mpairs * (a.num_col_tiles64 / 4u);
    const uint32_t pairs = std::min<uint32_t>(items, (uint32_t)num_sms / 2u);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * pairs, 1, 1);
    cfg.blockDim = dim3(kThreads + (ROWS ? 32 * kRowWarps : 0), 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k44_wave_umma_pair_kernel<ROWS>, tmap, wmap, a, d);
}

}  // namespace pairwave

cudaError_t launch_wave_umma_pair(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, const CUtensorMap &wmap, int num_sms, cudaStream_t s) {
    const uint32_t mtiles = (a.cout + kTileM - 1) / kTileM;
    if (a.gather_mode != GATHER_BOX || a.k_splits != 1u || !a.out_maps || a.cout_map || a.peers || (mtiles & 1u) || (a.mtiles_per_group & 1u) ||
        (a.num_col_tiles64 % 4u) != 0u)
        return cudaErrorInvalidValue;
    if (a.box_h == 1u) return pairwave::launch<1>(a, d, tmap, wmap, num_sms, s);
    if (a.box_h < 8u || 2u * (kStageK / a.box_h) > 32u) return cudaErrorInvalidValue;    // one producer lane per box
    return pairwave::launch<0>(a, d, tmap, wmap, num_sms, s);
}

}  // namespace k44b
