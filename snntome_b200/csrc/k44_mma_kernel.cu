// General wave kernel on the warp-level tensor path (mma.sync m16n8k16): any gather table (element-granular offsets,
// per-synapse token shifts), any group size that is a multiple of 16. It serves the waves tcgen05 cannot take — its
// smallest tile is 64 neurons sharing one operand, and its operand rows must be 16-byte aligned — i.e. the role of the
// reference's small-group and token-shift kernels (kernels/cuda/kernel44_cuda_pack.cuh:242-286). The FP32-FMA kernel
// stays as the arithmetic cross-check.
//
// CTA = 128 threads = MT x 16 neurons of one group (MT = 1, 2 or 4) x one 64-column tile; warp w owns columns
// 16w .. 16w+15. Per 64-synapse stage the gathered rows go to shared memory as [synapse][column] — with 16-byte loads
// where an offset is 16-byte aligned and unshifted, 2-byte loads with the causal mask otherwise — and the weight block
// as [neuron][synapse]; A fragments come from ldmatrix, B fragments from ldmatrix.trans (the tile is column-contiguous),
// FP32 accumulators in registers. Nothing here waits on anything.
#include "k44_kernels.cuh"
#include "k44_epilogue.cuh"

namespace k44b {
namespace mmawave {

constexpr uint32_t kPitch = 72;         // halves per shared-memory row (64 + 8: ldmatrix rows fall into distinct banks)

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int MT>
__global__ void __launch_bounds__(128) k44_wave_mma_kernel(const WaveArgs a) {
    __shared__ __align__(16) __half xs[kStageK][kPitch];
    __shared__ __align__(16) __half ws[MT * 16][kPitch];
    __shared__ uint64_t offs[kStageK];
    __shared__ uint32_t shs[kStageK];

    const uint32_t tile = blockIdx.x;                       // 64-column tile
    const uint32_t j0 = blockIdx.y * (MT * 16u);            // first neuron of this CTA
    const uint32_t g = j0 / a.group;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const __half *xbase = a.canvas + a.x_base_off + (uint64_t)tile * 64u;
    const uint64_t x_limit = a.canvas_elems - a.x_base_off - (uint64_t)tile * 64u;       // exclusive bound for off + 64
    const uint32_t flen = a.frame_len ? a.frame_len : a.pitch;
    const uint32_t tile_in_frame = (tile * 64u) % flen;

    float acc[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][n][e] = 0.f;
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
        }
        // weights: MT*16 rows x 8 vectors of 8 synapses
        for (uint32_t v = tid; v < MT * 16u * 8u; v += 128u) {
            const uint32_t r = v >> 3, k8 = v & 7u;
            uint4 wv = make_uint4(0u, 0u, 0u, 0u);
            if (j0 + r < a.cout) wv = a.w_tiles[tiled_vec_index(j0 + r, ks * 8u + k8, a.num_kstages)];
            *reinterpret_cast<uint4 *>(&ws[r][k8 * 8u]) = wv;
        }
        __syncthreads();
        // substrate rows: 64 synapses x 8 pieces of 8 columns
        for (uint32_t v = tid; v < kStageK * 8u; v += 128u) {
            const uint32_t k = v >> 3, piece = v & 7u;
            const uint64_t off = offs[k];
            const uint32_t sh = shs[k];
            const __half *src = xbase + off + piece * 8u;
            uint4 val;
            if (sh == 0u && ((a.x_base_off + off) & 7u) == 0u) {
                val = *reinterpret_cast<const uint4 *>(src);
            } else {
                __half h[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t cif = (tile_in_frame + piece * 8u + (uint32_t)e) % flen;        // column inside its frame
                    h[e] = cif >= sh ? src[(int)e - (int)sh] : __float2half(0.0f);
                }
                val = *reinterpret_cast<const uint4 *>(h);
            }
            *reinterpret_cast<uint4 *>(&xs[k][piece * 8u]) = val;
        }
        __syncthreads();
#pragma unroll
        for (uint32_t k16 = 0; k16 < kStageK / 16u; ++k16) {
            uint32_t bfrag[2][2];
#pragma unroll
            for (int n = 0; n < 2; ++n)
                ldmatrix_x2_trans(bfrag[n], (uint32_t)__cvta_generic_to_shared(&xs[k16 * 16u + (lane & 15u)][warp * 16u + (uint32_t)n * 8u]));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                uint32_t afrag[4];
                ldmatrix_x4(afrag, (uint32_t)__cvta_generic_to_shared(&ws[m * 16 + (lane & 15u)][k16 * 16u + (lane >> 4) * 8u]));
#pragma unroll
                for (int n = 0; n < 2; ++n) mma_16816(acc[m][n], afrag, bfrag[n]);
            }
        }
        __syncthreads();
    }
    if (bad) atomicOr(a.status, (uint32_t)ST_BAD_INDEX);

    // epilogue: accumulator (m, n): rows lane/4 and lane/4 + 8 of the 16-row block, columns (lane%4)*2 + {0,1} of the 8-column block
    const bool has_map = a.cout_map != nullptr;
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const uint32_t j = j0 + (uint32_t)m * 16u + (lane >> 2) + (uint32_t)hrow * 8u;
            if (j >= a.cout) continue;
            const uint32_t oj = has_map ? a.cout_map[j] : j;
            const float b = a.bias ? __half2float(a.bias[j]) : 0.0f;
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const uint64_t o = (uint64_t)oj * a.pitch + (uint64_t)tile * 64u + warp * 16u + (uint32_t)n * 8u + (lane & 3u) * 2u;
                float r0 = 0.f, r1 = 0.f;
                if (a.has_residual) {
                    const float2 rr = __half22float2(*reinterpret_cast<const __half2 *>(a.canvas + a.res_off + o));
                    r0 = rr.x; r1 = rr.y;
                }
                const float v0 = finish_value(acc[m][n][hrow * 2 + 0], b, r0, a.act, a.has_residual != 0, has_map);
                const float v1 = finish_value(acc[m][n][hrow * 2 + 1], b, r1, a.act, a.has_residual != 0, has_map);
                *reinterpret_cast<__half2 *>(a.canvas + a.y_off + o) = __floats2half2_rn(v0, v1);
            }
        }
}

}  // namespace mmawave

cudaError_t launch_wave_mma(const WaveArgs &a, cudaStream_t s) {
    if (a.group % 16u) return cudaErrorInvalidValue;
    // the CTA's neurons must share one gather list: 64, 32 or 16 of them, whichever divides the group
    const uint32_t rows = a.group % 64u == 0u ? 64u : (a.group % 32u == 0u ? 32u : 16u);
    const dim3 grid(a.num_col_tiles64, (a.cout + rows - 1u) / rows);
    switch (rows) {
    case 64: mmawave::k44_wave_mma_kernel<4><<<grid, 128, 0, s>>>(a); break;
    case 32: mmawave::k44_wave_mma_kernel<2><<<grid, 128, 0, s>>>(a); break;
    default: mmawave::k44_wave_mma_kernel<1><<<grid, 128, 0, s>>>(a); break;
    }
    return cudaGetLastError();
}

}  // namespace k44b
