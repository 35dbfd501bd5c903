// 2-D image glue between waves: commands that move or reduce pixels of haloed planes without any weights — 2x2 / stride-2 and
// 5x5 / stride-1 max-pooling, nearest-neighbour upsampling, space-to-depth (the polyphase split that turns a stride-2
// convolution into a stride-1 wave), the scatter that interleaves the four phase planes of a 2x2 transposed convolution,
// clearing of halos, and the dense F32 <-> plane conversions of the host boundary. Semantics follow
// kernels/common/kernel44_valu_pack.cuh:30-103; all of them are bound by memory traffic, so the kernels are plain
// grid-stride loops with consecutive threads on consecutive pixels of a row.
// Plane geometry: pixel (y, x) of a plane sits at (y + 1) * wpad + 4 + x (one halo row on top, four halo elements left).
#include "k44_kernels.cuh"

namespace k44b {

namespace {

__device__ __forceinline__ uint64_t px(uint32_t y, uint32_t x, uint32_t wpad) { return (uint64_t)(y + 1u) * wpad + 4u + x; }

// destination pixel (c, y, x) of an h_out x w_out image from a linear index
__device__ __forceinline__ void unpack(uint64_t i, uint32_t h, uint32_t w, uint32_t &c, uint32_t &y, uint32_t &x) {
    x = (uint32_t)(i % w);
    const uint64_t t = i / w;
    y = (uint32_t)(t % h);
    c = (uint32_t)(t / h);
}
// the same with several frames per channel: linear index over [plane][frame][y][x]
__device__ __forceinline__ void unpack(uint64_t i, uint32_t frames, uint32_t h, uint32_t w, uint32_t &c, uint32_t &f, uint32_t &y, uint32_t &x) {
    x = (uint32_t)(i % w);
    uint64_t t = i / w;
    y = (uint32_t)(t % h);
    t /= h;
    f = (uint32_t)(t % frames);
    c = (uint32_t)(t / frames);
}

__global__ void k44_image_maxpool2_kernel(const AuxArgs a) {
    const __half *src = a.canvas + a.src_off;
    __half *dst = a.canvas + a.dst_off;
    const uint64_t total = (uint64_t)a.rows * a.frames * a.h_out * a.w_out;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t c, f, y, x;
        unpack(i, a.frames, a.h_out, a.w_out, c, f, y, x);
        const __half *p = src + (uint64_t)c * a.cs_in + (uint64_t)f * a.fs_in + px(2u * y, 2u * x, a.wpad_in);
        const float m = fmaxf(fmaxf(__half2float(p[0]), __half2float(p[1])), fmaxf(__half2float(p[a.wpad_in]), __half2float(p[a.wpad_in + 1u])));
        dst[(uint64_t)c * a.cs_out + (uint64_t)f * a.fs_out + px(y, x, a.wpad_out)] = __float2half_rn(m);
    }
}

// window 5x5, stride 1, pad 2: pixels outside the image do not take part (they count as the most negative half)
__global__ void k44_image_maxpool5_kernel(const AuxArgs a) {
    const __half *src = a.canvas + a.src_off;
    __half *dst = a.canvas + a.dst_off;
    const uint64_t total = (uint64_t)a.rows * a.frames * a.h_out * a.w_out;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t c, f, y, x;
        unpack(i, a.frames, a.h_out, a.w_out, c, f, y, x);
        const __half *plane = src + (uint64_t)c * a.cs_in + (uint64_t)f * a.fs_in;
        float m = -65504.0f;
#pragma unroll
        for (int dy = -2; dy <= 2; ++dy) {
            const int yy = (int)y + dy;
            if (yy < 0 || yy >= (int)a.h_in) continue;
#pragma unroll
            for (int dx = -2; dx <= 2; ++dx) {
                const int xx = (int)x + dx;
                if (xx >= 0 && xx < (int)a.w_in) m = fmaxf(m, __half2float(plane[px((uint32_t)yy, (uint32_t)xx, a.wpad_in)]));
            }
        }
        dst[(uint64_t)c * a.cs_out + (uint64_t)f * a.fs_out + px(y, x, a.wpad_out)] = __float2half_rn(m);
    }
}

__global__ void k44_image_upsample2_kernel(const AuxArgs a) {
    const __half *src = a.canvas + a.src_off;
    __half *dst = a.canvas + a.dst_off;
    const uint64_t total = (uint64_t)a.rows * a.frames * a.h_out * a.w_out;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t c, f, y, x;
        unpack(i, a.frames, a.h_out, a.w_out, c, f, y, x);
        dst[(uint64_t)c * a.cs_out + (uint64_t)f * a.fs_out + px(y, x, a.wpad_out)] = src[(uint64_t)c * a.cs_in + (uint64_t)f * a.fs_in + px(y >> 1, x >> 1, a.wpad_in)];
    }
}

// input channel c -> four half-resolution planes 4c + 2*py + px holding the pixels of row parity py and column parity px
__global__ void k44_image_s2d_kernel(const AuxArgs a) {
    const __half *src = a.canvas + a.src_off;
    __half *dst = a.canvas + a.dst_off;
    const uint64_t total = (uint64_t)a.rows * 4u * a.frames * a.h_out * a.w_out;         // a.rows = input channels
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t c4, f, y, x;
        unpack(i, a.frames, a.h_out, a.w_out, c4, f, y, x);
        const uint32_t c = c4 >> 2, py = (c4 >> 1) & 1u, pxx = c4 & 1u;
        dst[(uint64_t)c4 * a.cs_out + (uint64_t)f * a.fs_out + px(y, x, a.wpad_out)] = src[(uint64_t)c * a.cs_in + (uint64_t)f * a.fs_in + px(2u * y + py, 2u * x + pxx, a.wpad_in)];
    }
}

// the wave of a 2x2 / stride-2 transposed convolution writes, at input resolution, plane q * rows + c for output phase
// q = 2 * (y & 1) + (x & 1); this interleaves the four phases into the full-resolution tensor
__global__ void k44_image_upconv_scatter_kernel(const AuxArgs a) {
    const __half *src = a.canvas + a.src_off;
    __half *dst = a.canvas + a.dst_off;
    const uint64_t total = (uint64_t)a.rows * a.frames * a.h_out * a.w_out;              // a.rows = output channels
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t c, f, y, x;
        unpack(i, a.frames, a.h_out, a.w_out, c, f, y, x);
        const uint32_t q = ((y & 1u) << 1) | (x & 1u);
        dst[(uint64_t)c * a.cs_out + (uint64_t)f * a.fs_out + px(y, x, a.wpad_out)] = src[(uint64_t)(q * a.rows + c) * a.cs_in + (uint64_t)f * a.fs_in + px(y >> 1, x >> 1, a.wpad_in)];
    }
}

// everything of the `rows` planes at dst that is not a pixel becomes zero
__global__ void k44_image_halo_clear_kernel(const AuxArgs a) {
    __half *dst = a.canvas + a.dst_off;
    const uint64_t total = (uint64_t)a.rows * a.cs_out;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t e = (uint32_t)(i % a.cs_out) % a.fs_out;        // element inside its frame
        const uint32_t row = e / a.wpad_out, col = e % a.wpad_out;
        const bool pixel = row >= 1u && row <= a.h_out && col >= 4u && col < 4u + a.w_out;
        if (!pixel) dst[i] = __float2half(0.0f);
    }
}

// dense [frame][channel][y][x] FP32 at the host boundary <-> planes (channel-major, the frames of a channel side by side)
__global__ void k44_f32_to_planes_kernel(const float *__restrict__ src, __half *__restrict__ dst, uint32_t channels, uint32_t h, uint32_t w, uint32_t wpad, uint32_t cs,
                                         uint32_t fs, uint64_t total) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t f, c, y, x;
        unpack(i, channels, h, w, f, c, y, x);
        dst[(uint64_t)c * cs + (uint64_t)f * fs + px(y, x, wpad)] = __float2half_rn(src[i]);
    }
}

__global__ void k44_planes_to_f32_kernel(const __half *__restrict__ src, float *__restrict__ dst, uint32_t channels, uint32_t h, uint32_t w, uint32_t wpad, uint32_t cs,
                                         uint32_t fs, uint64_t total) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t f, c, y, x;
        unpack(i, channels, h, w, f, c, y, x);
        dst[i] = __half2float(src[(uint64_t)c * cs + (uint64_t)f * fs + px(y, x, wpad)]);
    }
}

inline uint32_t grid_of(uint64_t total) {
    const uint64_t g = (total + 255u) / 256u;
    return (uint32_t)(g < 148ull * 16ull ? (g ? g : 1) : 148ull * 16ull);
}

}  // namespace

cudaError_t launch_image_aux(const AuxArgs &a, cudaStream_t s) {
    if (!a.rows || !a.h_out || !a.w_out || !a.wpad_out || !a.cs_out || !a.frames || !a.fs_out) return cudaErrorInvalidValue;
    const uint64_t out_px = (uint64_t)a.rows * a.frames * a.h_out * a.w_out;
    switch (a.kind) {
    case AUX_MAXPOOL2: k44_image_maxpool2_kernel<<<grid_of(out_px), 256, 0, s>>>(a); break;
    case AUX_MAXPOOL5: k44_image_maxpool5_kernel<<<grid_of(out_px), 256, 0, s>>>(a); break;
    case AUX_UPSAMPLE2: k44_image_upsample2_kernel<<<grid_of(out_px), 256, 0, s>>>(a); break;
    case AUX_S2D: k44_image_s2d_kernel<<<grid_of(out_px * 4u), 256, 0, s>>>(a); break;
    case AUX_UPCONV_SCATTER: k44_image_upconv_scatter_kernel<<<grid_of(out_px), 256, 0, s>>>(a); break;
    case AUX_HALO_CLEAR: k44_image_halo_clear_kernel<<<grid_of((uint64_t)a.rows * a.cs_out), 256, 0, s>>>(a); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_f32_to_planes(const float *src, __half *dst, uint32_t c, uint32_t h, uint32_t w, uint32_t wpad, uint32_t cs, uint32_t frames, uint32_t fs, cudaStream_t s) {
    const uint64_t total = (uint64_t)frames * c * h * w;
    k44_f32_to_planes_kernel<<<grid_of(total), 256, 0, s>>>(src, dst, c, h, w, wpad, cs, fs, total);
    return cudaGetLastError();
}

cudaError_t launch_planes_to_f32(const __half *src, float *dst, uint32_t c, uint32_t h, uint32_t w, uint32_t wpad, uint32_t cs, uint32_t frames, uint32_t fs, cudaStream_t s) {
    const uint64_t total = (uint64_t)frames * c * h * w;
    k44_planes_to_f32_kernel<<<grid_of(total), 256, 0, s>>>(src, dst, c, h, w, wpad, cs, fs, total);
    return cudaGetLastError();
}

}  // namespace k44b
