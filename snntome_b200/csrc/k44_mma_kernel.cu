// General wave kernel on the warp-level tensor path (mma.sync m16n8k16): any gather table (element-granular offsets,
// per-synapse token shifts), any group size that is a multiple of 16. It serves the waves tcgen05 cannot take — its
// smallest tile is 64 neurons sharing one operand, and its operand rows must be 16-byte aligned — i.e. the role of the
// reference's small-group and token-shift kernels (kernels/cuda/kernel44_cuda_pack.cuh:242-286). The FP32-FMA kernel
// stays as the arithmetic cross-check.
//
// CTA = 128 threads = MT x 16 neurons of one group (MT = 1, 2 or 4) x one 64-column tile; warp w owns columns
// 16w .. 16w+15 (64 rows: the four warps form a 2 x 2 grid of 32 x 32 blocks). A ring of kStages (two) stages of 64 synapses is filled with cp.async: the gathered rows as [synapse][column]
// (row pitch 72 halves, so the 8 rows of an ldmatrix fall into distinct banks) and the weight rows exactly as the tiled
// format stores them (128-byte rows, 16-byte chunk c at position c ^ (row & 7): conflict-free for ldmatrix as it is).
// Gather-table entries travel two stages ahead of their rows in a small ring of their own. Rows whose offset is not
// 16-byte aligned, or that carry a token shift, are cut out of the two aligned 16-byte vectors around them (funnel shift,
// causal mask in registers) by the same thread that would have issued the copy. A fragments come from ldmatrix, B fragments from ldmatrix.trans, FP32 accumulators in
// registers. Nothing here waits on another CTA; in a neuron-sharded plan one thread waits (bounded) for the peer GPUs' previous
// launches before the first gather, every output pair is also stored into the peers' canvases, and the CTA that finishes
// last publishes the launch count (same protocol as the tcgen05 kernels).
#include <cstdlib>
#include "k44_kernels.cuh"
#include "k44_epilogue.cuh"

namespace k44b {
namespace mmawave {

constexpr uint32_t kPitch = 72;         // halves per gathered row in shared memory
constexpr uint32_t kStages = 2;          // measured: six CTAs per SM with two stages beat four CTAs with three (0.91 vs 0.75 of the HBM rate at 64 rows)
constexpr uint32_t kXBytesStage = kStageK * kPitch * 2u;
constexpr uint32_t kTabRing = 2u * (kStages - 1u) + 1u;   // table entries run up to 2 (kStages - 1) stages ahead of the stage being consumed
constexpr uint32_t smem_bytes(uint32_t mt) { return kStages * (kXBytesStage + mt * 16u * 128u) + kTabRing * kStageK * 4u; }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Eight columns of a gathered row whose start is not 16-byte aligned or that carries a token shift are cut out of the two
// aligned 16-byte vectors around them (funnel shift); columns whose position inside their frame is below the shift read
// zero.
// `elem` is the canvas element of the unshifted first column, `cif0` that column's position inside its frame.
__device__ __forceinline__ bool unaligned_in_range(uint64_t canvas_elems, uint64_t elem, uint32_t sh) {
    return elem >= sh && ((elem - sh) & ~7ull) + 16u <= canvas_elems;
}
__device__ __forceinline__ uint4 finish_unaligned(const uint4 &v0, const uint4 &v1, uint32_t m, uint32_t sh, uint32_t cif0, uint32_t flen) {
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    const uint32_t bits = (m & 1u) * 16u;
    uint32_t out[4];
    switch (m >> 1) {
    case 0:
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = __funnelshift_r(w[i], w[i + 1], bits);
        break;
    case 1:
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = __funnelshift_r(w[i + 1], w[i + 2], bits);
        break;
    case 2:
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = __funnelshift_r(w[i + 2], w[i + 3], bits);
        break;
    default:
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = __funnelshift_r(w[i + 3], w[i + 4], bits);
        break;
    }
    if (sh != 0u && !(cif0 >= sh && cif0 + 7u < flen)) {       // some of the eight columns sit left of their frame's column `sh`
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t cif = (cif0 + (uint32_t)c) % flen;
            if (cif < sh) out[c >> 1] &= (c & 1) ? 0x0000ffffu : 0xffff0000u;
        }
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}
// the same at the very edge of the canvas, element by element
__device__ __forceinline__ uint4 fetch_piece_edge(const __half *canvas, uint64_t canvas_elems, uint64_t elem, uint32_t sh, uint32_t cif0, uint32_t flen) {
    __half h[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const uint32_t cif = (cif0 + (uint32_t)c) % flen;
        const uint64_t e = elem + (uint64_t)c;
        h[c] = (cif >= sh && e >= sh && e - sh < canvas_elems) ? canvas[e - sh] : __float2half(0.0f);
    }
    return *reinterpret_cast<const uint4 *>(h);
}

template <int MT>
__global__ void __launch_bounds__(128) k44_wave_mma_kernel(const WaveArgs a, const unsigned long long wait_cycles) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t kWBytesStage = MT * 16u * 128u;
    constexpr uint32_t D = kStages - 1u;                    // stages in flight ahead of the one being consumed
    const uint32_t xs = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t ws = xs + kStages * kXBytesStage;
    const uint32_t tabs = ws + kStages * kWBytesStage;
    uint8_t *const xs_gen = smem;
    const uint32_t *const tab_gen = reinterpret_cast<const uint32_t *>(smem + kStages * (kXBytesStage + kWBytesStage));

    // one-dimensional grid (the y extent of a grid stops at 65535 blocks: too few for a million neurons in blocks of 16);
    // column tiles of one neuron block are neighbours, so they find the block's weights in L2
    const uint32_t tile = blockIdx.x % a.num_col_tiles64;                   // 64-column tile
    const uint32_t j0 = (blockIdx.x / a.num_col_tiles64) * (MT * 16u);      // first neuron of this CTA
    const uint32_t g = j0 / a.group;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint64_t tile_x = a.tile_off_x ? a.tile_off_x[tile] : (uint64_t)tile * 64u;          // where this tile's gathers are anchored (2-D planes: a table)
    const __half *xbase = a.canvas + a.x_base_off + tile_x;
    const uint64_t x_limit = a.canvas_elems - a.x_base_off - tile_x;       // exclusive bound for off + 64
    const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
    const uint32_t tile_in_frame = (tile * 64u) % flen;
    const uint32_t nk = a.num_kstages;
    const bool box = a.gather_mode == GATHER_BOX;
    const uint32_t *table = a.gather + (uint64_t)g * (box ? a.boxes_per_group : a.fan_in);
    const uint4 *wrow0 = a.w_tiles + ((uint64_t)(j0 >> 7) * nk * 128u + (j0 & 127u)) * 8u;   // + ks * 1024 vectors per stage

    // warp grid: 2 x 2 warps for 64 rows (each warp: two 16-row blocks x 32 columns), 1 x 4 for 16 / 32 rows (all rows x 16
    // columns per warp; measured: 2 x 2 gains 2 % at 64 rows and loses 8 % at 32). The B fragments of two neighbouring
    // 8-column blocks come from one ldmatrix.x4.trans and are reused by the warp's MW row blocks.
    constexpr uint32_t WR = MT >= 4 ? 2u : 1u, WC = 4u / WR, MW = MT / WR, NW = 8u / WC;
    const uint32_t wr = warp / WC, wc = warp % WC;
    float acc[MW][NW][4];
#pragma unroll
    for (int m = 0; m < (int)MW; ++m)
#pragma unroll
        for (int n = 0; n < (int)NW; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.f;
    bool bad = false;

    // table entry of synapse tid of stage ks (clamped to the last real synapse: its weight is zero past fan_in)
    const uint32_t piece = tid & 7u;
    const uint32_t cif0 = (tile_in_frame + piece * 8u) % flen;
    const uint32_t box_mask = a.box_h - 1u, box_shift = 31u - (uint32_t)__clz((int)(a.box_h | 1u));   // box heights are powers of two
    auto issue_table = [&](uint32_t ks) {
        if (tid < kStageK && ks < nk) {
            const uint32_t s = min(ks * kStageK + tid, a.fan_in - 1u);
            cp_async_4(tabs + ((ks % kTabRing) * kStageK + tid) * 4u, table + (box ? s >> box_shift : s));
        }
    };
    auto issue_data = [&](uint32_t ks) {
        if (ks >= nk) return;
        const uint32_t st = ks % kStages;
        // weights: MT*16 rows of 128 bytes, contiguous in the tiled format
        const uint4 *wsrc = wrow0 + (uint64_t)ks * 1024u;
#pragma unroll
        for (uint32_t v = tid; v < MT * 128u; v += 128u) cp_async_16(ws + st * kWBytesStage + v * 16u, wsrc + v);
        // gathered rows: 64 synapses x 8 pieces of 8 columns
#pragma unroll
        for (uint32_t i = 0; i < 4u; ++i) {
            const uint32_t k = (tid >> 3) + 16u * i;
            const uint32_t s = min(ks * kStageK + k, a.fan_in - 1u);
            const uint32_t e = tab_gen[(ks % kTabRing) * kStageK + k];
            uint64_t off;
            uint32_t sh;
            if (box) { off = (uint64_t)((e & kBoxRowMask) + (s & box_mask)) * a.pitch; sh = e >> 28; }
            else { off = e; sh = a.shifts ? a.shifts[(uint64_t)g * a.fan_in + s] : 0u; }
            if (off + 64u > x_limit) { off = 0; bad = true; }   // record and skip instead of faulting
            const uint32_t dst_off = st * kXBytesStage + (k * kPitch + piece * 8u) * 2u;
            if (sh == 0u && ((a.x_base_off + tile_x + off) & 7u) == 0u) {
                cp_async_16(xs + dst_off, xbase + off + piece * 8u);
            } else {
                const uint64_t elem = a.x_base_off + tile_x + off + piece * 8u;
                uint4 val;
                if (unaligned_in_range(a.canvas_elems, elem, sh)) {
                    const uint64_t first = elem - sh, lo = first & ~7ull;
                    const uint32_t m = (uint32_t)(first - lo);
                    const uint4 v0 = *reinterpret_cast<const uint4 *>(a.canvas + lo);
                    const uint4 v1 = m ? *reinterpret_cast<const uint4 *>(a.canvas + lo + 8u) : v0;
                    val = finish_unaligned(v0, v1, m, sh, cif0, flen);
                } else {
                    val = fetch_piece_edge(a.canvas, a.canvas_elems, elem, sh, cif0, flen);
                }
                *reinterpret_cast<uint4 *>(xs_gen + dst_off) = val;
            }
        }
    };

    // neuron-sharded plans: the rows this launch gathers were stored into this canvas by the peers' previous launches
    // (the grid is not persistent: once one CTA has given up on a peer, the status bit tells every later CTA not to wait
    // again, so a missing peer costs one wait period and not one per batch of resident CTAs; a launch that gave up reads and
    // stores nothing and only counts its CTAs as done)
    bool peers_ready = true;
    if (a.peers) {
        __shared__ uint32_t peer_ok;
        if (tid == 0) {
            uint32_t ok = (*reinterpret_cast<volatile uint32_t *>(a.status) & (uint32_t)ST_TIMEOUT_PEER) ? 0u : 1u;
            if (ok) ok = peer_wait_ready(a.peers, wait_cycles, a.peer_slack) ? 1u : 0u;
            if (!ok) atomicOr(a.status, (uint32_t)ST_TIMEOUT_PEER);
            peer_ok = ok;
        }
        __syncthreads();
        peers_ready = peer_ok != 0u;
    }
    if (peers_ready) {

    // prologue: table entries of the first 2D stages, then the rows of the first D stages
    for (uint32_t ks = 0; ks < 2u * D; ++ks) issue_table(ks);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    for (uint32_t ks = 0; ks < D; ++ks) { issue_data(ks); cp_async_commit(); }

    for (uint32_t ks = 0; ks < nk; ++ks) {
        cp_async_wait<D - 1>();             // rows of stage ks (and the table entries of stage ks + D) have landed
        __syncthreads();                    // ... for every thread; and everyone is done with the stage refilled below
        issue_data(ks + D);
        issue_table(ks + 2u * D);
        cp_async_commit();
        const uint32_t st = ks % kStages;
        const uint32_t xs_st = xs + st * kXBytesStage, ws_st = ws + st * kWBytesStage;
#pragma unroll
        for (uint32_t k16 = 0; k16 < kStageK / 16u; ++k16) {
            uint32_t bfrag[NW][2];
#pragma unroll
            for (int n2 = 0; n2 < (int)NW / 2; ++n2) {
                // four 8 x 8 blocks: synapses 0-7 / 8-15 of this K step x two neighbouring 8-column blocks
                uint32_t t4[4];
                ldmatrix_x4_trans(t4, xs_st + ((k16 * 16u + (lane & 15u)) * kPitch + wc * (NW * 8u) + (uint32_t)n2 * 16u + (lane >> 4) * 8u) * 2u);
                bfrag[2 * n2][0] = t4[0]; bfrag[2 * n2][1] = t4[1];
                bfrag[2 * n2 + 1][0] = t4[2]; bfrag[2 * n2 + 1][1] = t4[3];
            }
#pragma unroll
            for (int m = 0; m < (int)MW; ++m) {
                uint32_t afrag[4];
                const uint32_t r = (wr * MW + (uint32_t)m) * 16u + (lane & 15u);
                // the tile's swizzle uses the row inside the 128-row tile; j0 is a multiple of 16, so (j0 + r) & 7 == r & 7
                ldmatrix_x4(afrag, ws_st + r * 128u + (((k16 * 2u + (lane >> 4)) ^ (r & 7u)) << 4));
#pragma unroll
                for (int n = 0; n < (int)NW; ++n) mma_16816(acc[m][n], afrag, bfrag[n]);
            }
        }
    }
    cp_async_wait<0>();
    if (bad) atomicOr(a.status, (uint32_t)ST_BAD_INDEX);

    // epilogue: accumulator (m, n): rows lane/4 and lane/4 + 8 of the 16-row block, columns (lane%4)*2 + {0,1} of the 8-column
    // block. The finished values are parked in shared memory (the gather ring is free by now) and leave as whole 16-byte
    // pieces, 128 contiguous bytes per row — to this canvas and, in a sharded plan, to every peer's.
    const bool has_map = a.cout_map != nullptr;
    uint64_t tile_y = (uint64_t)tile * 64u;                 // where this tile's outputs go inside a row / plane
    uint32_t quad_mask = 0xffffu;
    if (a.tile_off_y) {
        const uint32_t e = a.tile_off_y[tile];
        tile_y = a.tile_mask ? (uint64_t)(e & 0xffffu) << 2 : e;
        if (a.tile_mask) quad_mask = e >> 16;
    }
    __syncthreads();                        // every warp is done reading the last stage
    __half *const tile_out = reinterpret_cast<__half *>(xs_gen);       // [MT * 16][kPitch]
#pragma unroll
    for (int m = 0; m < (int)MW; ++m)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const uint32_t rl = (wr * MW + (uint32_t)m) * 16u + (lane >> 2) + (uint32_t)hrow * 8u;
            const uint32_t j = j0 + rl;
            if (j >= a.cout) continue;
            const uint32_t oj = has_map ? a.cout_map[j] : j;
            const float b = a.bias ? __half2float(a.bias[j]) : 0.0f;
#pragma unroll
            for (int n = 0; n < (int)NW; ++n) {
                const uint32_t col = wc * (NW * 8u) + (uint32_t)n * 8u + (lane & 3u) * 2u;
                float r0 = 0.f, r1 = 0.f;
                if (a.has_residual) {
                    const float2 rr = __half22float2(*reinterpret_cast<const __half2 *>(a.canvas + a.res_off + (uint64_t)oj * a.pitch + tile_y + col));
                    r0 = rr.x; r1 = rr.y;
                }
                const float v0 = finish_value(acc[m][n][hrow * 2 + 0], b, r0, a.act, a.has_residual != 0, has_map);
                const float v1 = finish_value(acc[m][n][hrow * 2 + 1], b, r1, a.act, a.has_residual != 0, has_map);
                *reinterpret_cast<__half2 *>(tile_out + rl * kPitch + col) = __floats2half2_rn(v0, v1);
            }
        }
    __syncthreads();
    if (a.tile_off_y) {
        // 2-D planes: tiles start on 8-byte boundaries only and may cover halo elements: 4-element quads, masked
#pragma unroll
        for (uint32_t p = tid; p < MT * 16u * 16u; p += 128u) {
            const uint32_t rl = p >> 4, qd = p & 15u;
            const uint32_t j = j0 + rl;
            if (j >= a.cout || !((quad_mask >> qd) & 1u)) continue;
            const uint32_t oj = has_map ? a.cout_map[j] : j;
            *reinterpret_cast<uint2 *>(a.canvas + a.y_off + (uint64_t)oj * a.pitch + tile_y + qd * 4u) =
                *reinterpret_cast<const uint2 *>(tile_out + rl * kPitch + qd * 4u);
        }
    } else {
#pragma unroll
    for (uint32_t p = tid; p < MT * 16u * 8u; p += 128u) {
        const uint32_t rl = p >> 3, pc = p & 7u;
        const uint32_t j = j0 + rl;
        if (j >= a.cout) continue;
        const uint32_t oj = has_map ? a.cout_map[j] : j;
        const uint64_t off = a.y_off + (uint64_t)oj * a.pitch + (uint64_t)tile * 64u + pc * 8u;
        const uint4 val = *reinterpret_cast<const uint4 *>(tile_out + rl * kPitch + pc * 8u);
        *reinterpret_cast<uint4 *>(a.canvas + off) = val;
        if (a.peers) store_to_peers(a.peers, off, val);
    }
    }
    }   // peers_ready
    if (a.peers) {
        __syncthreads();                    // orders every thread's peer stores before thread 0's system-scope fence
        if (tid == 0) peer_signal_done(a.peers, gridDim.x);
    }
}

}  // namespace mmawave

cudaError_t launch_wave_mma(const WaveArgs &a, unsigned long long wait_cycles, cudaStream_t s) {
    if (a.group % 16u) return cudaErrorInvalidValue;
    // the CTA's neurons must share one gather list: 64, 32 or 16 of them, whichever divides the group
    uint32_t rows = a.group % 64u == 0u ? 64u : (a.group % 32u == 0u ? 32u : 16u);
    // a wave with fewer CTAs than four per SM (the deep layers of an image network: a 20 x 20 map is 7 pixel tiles)
    // is cut into smaller neuron blocks: each CTA gathers the same rows again, but they come out of L2 and the wave's time
    // is its longest CTA's K loop, not its bytes
    static const uint64_t min_blocks = [] { const char *e = std::getenv("K44B_MMA_MIN_BLOCKS"); const long v = e ? std::atol(e) : 0; return v > 0 ? (uint64_t)v : 592ull; }();
    while (rows > 16u && (uint64_t)a.num_col_tiles64 * ((a.cout + rows - 1u) / rows) < min_blocks) rows >>= 1;
    const uint64_t blocks = (uint64_t)a.num_col_tiles64 * ((a.cout + rows - 1u) / rows);
    if (blocks == 0 || blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    const dim3 grid((uint32_t)blocks);
    switch (rows) {
    case 64: mmawave::k44_wave_mma_kernel<4><<<grid, 128, mmawave::smem_bytes(4), s>>>(a, wait_cycles); break;
    case 32: mmawave::k44_wave_mma_kernel<2><<<grid, 128, mmawave::smem_bytes(2), s>>>(a, wait_cycles); break;
    default: mmawave::k44_wave_mma_kernel<1><<<grid, 128, mmawave::smem_bytes(1), s>>>(a, wait_cycles); break;
    }
    return cudaGetLastError();
}

cudaError_t mma_kernel_setup() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(mmawave::k44_wave_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mmawave::smem_bytes(4))) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(mmawave::k44_wave_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mmawave::smem_bytes(2))) != cudaSuccess) return e;
    return cudaFuncSetAttribute(mmawave::k44_wave_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mmawave::smem_bytes(1));
}

}  // namespace k44b
