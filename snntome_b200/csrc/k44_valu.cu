// Element-wise and attention steps between the waves of a decoder layer, on the 1-D token layout (channel-major:
// channel c of a tensor at element offset `off` is canvas[off + c*pitch ...]). All of them are bandwidth- or
// latency-bound SIMT kernels; none is on the tensor cores.
//
//   RMSNorm        y[c][t] = x[c][t] * rsqrt(mean_c x[c][t]^2 + eps) * gamma[c]      (kernels/common/kernel44_valu_pack.cuh:104-134)
//   SwiGLU product y = gate * up (SiLU is applied by the gate wave's epilogue)          (:135-143)
//   rotary         pairs (p, p + head_dim/2), angle = position * theta^(-2p/head_dim)  (:65-70, 144-158)
//   causal GQA     per sequence of `seq_len` columns, streaming softmax                (:159-248)
//   decode GQA     one new token per column against a key / value cache in the canvas  (no counterpart in the reference)
//
// FP16 in and out, FP32 arithmetic, one rounding (to nearest even) at each store, as the reference kernels do.
#include "k44_kernels.cuh"

namespace k44b {

// Every kernel here may be launched with programmatic stream serialisation: it lets the next kernel start its own set-up
// at once and waits itself for the previous kernel's results before touching memory.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, bool pdl, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ void unpack8(const uint4 &u, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 v = __half22float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __half2 *h = reinterpret_cast<__half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return u;
}

// ---- RMSNorm: one CTA of 1024 threads per group of 8 columns ------------------------------------------------------------
// Thread t owns channels t, t + 1024, ...; with at most R of them per thread the 16-byte pieces stay in registers between
// the sum of squares and the scaling, so the tensor is read once and all loads of a thread are in flight together (a decode
// step has only 8 such CTAs, so latency, not bandwidth, is what counts). Larger tensors take the two-pass loop (R = 0).
template <int R>
__global__ void __launch_bounds__(1024) k44_valu_rmsnorm_kernel(const AuxArgs a) {
    pdl_enter();
    __shared__ float part[32][8];
    __shared__ float inv_s[8];
    const uint32_t col0 = blockIdx.x * 8u, tid = threadIdx.x;
    const __half *src = a.canvas + a.src_off + col0;
    __half *dst = a.canvas + a.dst_off + col0;
    float ss[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 keep[R > 0 ? R : 1];
    if (R > 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t c = tid + 1024u * (uint32_t)r;
            keep[r] = c < a.rows ? *reinterpret_cast<const uint4 *>(src + (uint64_t)c * a.pitch) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float x[8];
            unpack8(keep[r], x);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss[k] = fmaf(x[k], x[k], ss[k]);
        }
    } else {
        for (uint32_t c = tid; c < a.rows; c += 1024u) {
            float x[8];
            unpack8(*reinterpret_cast<const uint4 *>(src + (uint64_t)c * a.pitch), x);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss[k] = fmaf(x[k], x[k], ss[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss[k] += __shfl_xor_sync(0xffffffffu, ss[k], o);
    }
    if ((tid & 31u) == 0u) {
#pragma unroll
        for (int k = 0; k < 8; ++k) part[tid >> 5][k] = ss[k];
    }
    __syncthreads();
    if (tid < 32u) {                                   // one warp folds the 32 per-warp sums and publishes 1/rms per column
        const float inv_d = 1.0f / (float)a.rows;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float tot = part[tid][k];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
            if (tid == 0u) inv_s[k] = rsqrtf(fmaf(tot, inv_d, a.eps));
        }
    }
    __syncthreads();
    float inv[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) inv[k] = inv_s[k];
    if (R > 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t c = tid + 1024u * (uint32_t)r;
            if (c >= a.rows) break;
            float x[8];
            unpack8(keep[r], x);
            const float g = a.gamma ? __half2float(a.gamma[c]) : 1.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) x[k] = x[k] * inv[k] * g;
            *reinterpret_cast<uint4 *>(dst + (uint64_t)c * a.pitch) = pack8(x);
        }
    } else {
        for (uint32_t c = tid; c < a.rows; c += 1024u) {      // second pass: the rows come back from L2
            float x[8];
            unpack8(*reinterpret_cast<const uint4 *>(src + (uint64_t)c * a.pitch), x);
            const float g = a.gamma ? __half2float(a.gamma[c]) : 1.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) x[k] = x[k] * inv[k] * g;
            *reinterpret_cast<uint4 *>(dst + (uint64_t)c * a.pitch) = pack8(x);
        }
    }
}

// ---- SwiGLU product ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k44_valu_swiglu_kernel(const AuxArgs a) {
    pdl_enter();
    const uint64_t n8 = (uint64_t)a.rows * a.pitch / 8u;
    const uint4 *g = reinterpret_cast<const uint4 *>(a.canvas + a.src_off);
    const uint4 *u = reinterpret_cast<const uint4 *>(a.canvas + a.src2_off);
    uint4 *d = reinterpret_cast<uint4 *>(a.canvas + a.dst_off);
    for (uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x; i < n8; i += (uint64_t)gridDim.x * 256u) {
        float x[8], y[8];
        unpack8(g[i], x);
        unpack8(u[i], y);
#pragma unroll
        for (int k = 0; k < 8; ++k) x[k] *= y[k];
        d[i] = pack8(x);
    }
}

// ---- rotary embedding, in place -------------------------------------------------------------------------------------
__device__ __forceinline__ float rope_inv_freq(uint32_t p, uint32_t head_dim, float neg_log_theta, bool llama3) {
    float f = expf((float)(2u * p) * (neg_log_theta / (float)head_dim));
    if (llama3) {       // Llama-3 long-context frequency scaling
        const float ratio = 1303.7972938088068f * f;
        const float smooth = fminf(1.0f, fmaxf(0.0f, (ratio - 1.0f) * 0.3333333432674408f));
        f = (1.0f - smooth) * (f * 0.03125f) + smooth * f;
    }
    return f;
}

// one thread: one rotation pair of one head, 8 consecutive columns
__global__ void __launch_bounds__(256) k44_valu_rope_kernel(const AuxArgs a, uint64_t off, uint32_t heads) {
    pdl_enter();
    const uint32_t half = a.head_dim / 2u, groups = a.pitch / 8u;
    const uint64_t total = (uint64_t)heads * half * groups;
    const uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    if (i >= total) return;
    const uint32_t cg = (uint32_t)(i % groups);
    const uint32_t p = (uint32_t)((i / groups) % half), h = (uint32_t)(i / ((uint64_t)groups * half));
    __half *r0 = a.canvas + off + (uint64_t)(h * a.head_dim + p) * a.pitch + cg * 8u;
    __half *r1 = r0 + (uint64_t)half * a.pitch;
    const float f = rope_inv_freq(p, a.head_dim, a.neg_log_theta, a.llama3 != 0u);
    float x0[8], x1[8];
    unpack8(*reinterpret_cast<const uint4 *>(r0), x0);
    unpack8(*reinterpret_cast<const uint4 *>(r1), x1);
    const int fixed_pos = a.pos_ptr ? *a.pos_ptr : -1;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint32_t t = cg * 8u + (uint32_t)k;
        const float pos = fixed_pos >= 0 ? (float)fixed_pos : (float)(t % a.seq_len);
        float s, c;
        sincosf(pos * f, &s, &c);
        const float y0 = x0[k] * c - x1[k] * s, y1 = x0[k] * s + x1[k] * c;
        x0[k] = y0; x1[k] = y1;
    }
    *reinterpret_cast<uint4 *>(r0) = pack8(x0);
    *reinterpret_cast<uint4 *>(r1) = pack8(x1);
}

// ---- causal grouped-query attention ---------------------------------------------------------------------------------
// CTA = 32 consecutive columns (queries) of one query head; 4 threads per query, each owning HD/4 dimensions.
// Keys and values are visited in tiles of 32 columns from the start of the query's sequence, staged through shared
// memory as [column][dimension]; running maximum / sum softmax in FP32.
template <int HD>
__global__ void __launch_bounds__(128) k44_valu_causal_attn_kernel(const AuxArgs a) {
    pdl_enter();
    constexpr int DP = HD / 4;                      // dimensions per thread
    constexpr int ROW = HD + 8;                     // padded shared row (halves)
    __shared__ __align__(16) __half sk[32][ROW];
    __shared__ __align__(16) __half sv[32][ROW];
    const uint32_t tile = blockIdx.x, hq = blockIdx.y, hkv = hq / (a.h_q / a.h_kv);
    const uint32_t tid = threadIdx.x, part = tid & 3u, ql = tid >> 2;
    const uint32_t t0 = tile * 32u, t = t0 + ql;
    const uint32_t seq0 = (t0 / a.seq_len) * a.seq_len;           // first column of this sequence
    const float scale = rsqrtf((float)HD);
    const __half *qh = a.canvas + a.src_off + (uint64_t)hq * HD * a.pitch;
    const __half *kh = a.canvas + a.src2_off + (uint64_t)hkv * HD * a.pitch;
    const __half *vh = a.canvas + a.src3_off + (uint64_t)hkv * HD * a.pitch;
    // stage the query tile (coalesced rows of 32 columns), then keep this thread's slice in registers
    for (uint32_t e = tid; e < 32u * HD; e += 128u) { const uint32_t d = e >> 5, c = e & 31u; sk[c][d] = qh[(uint64_t)d * a.pitch + t0 + c]; }
    __syncthreads();
    float q[DP], acc[DP];
#pragma unroll
    for (int d = 0; d < DP; ++d) { q[d] = __half2float(sk[ql][part * DP + d]) * scale; acc[d] = 0.f; }
    __syncthreads();
    float m = -65504.0f, l = 0.f;
    for (uint32_t k0 = seq0; k0 <= t0; k0 += 32u) {
        for (uint32_t e = tid; e < 32u * HD; e += 128u) {
            const uint32_t d = e >> 5, c = e & 31u;
            sk[c][d] = kh[(uint64_t)d * a.pitch + k0 + c];
            sv[c][d] = vh[(uint64_t)d * a.pitch + k0 + c];
        }
        __syncthreads();
        const uint32_t last = (k0 == t0) ? ql : 31u;              // causal: keys up to the query's own column
        for (uint32_t u = 0; u <= 31u; ++u) {
            float dot = 0.f;
#pragma unroll
            for (int d = 0; d < DP; ++d) dot = fmaf(q[d], __half2float(sk[u][part * DP + d]), dot);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (u <= last) {
                const float mn = fmaxf(m, dot);
                const float ep = __expf(m - mn), ec = __expf(dot - mn);
                l = l * ep + ec;
#pragma unroll
                for (int d = 0; d < DP; ++d) acc[d] = acc[d] * ep + ec * __half2float(sv[u][part * DP + d]);
                m = mn;
            }
        }
        __syncthreads();
    }
    const float inv_l = 1.0f / l;
#pragma unroll
    for (int d = 0; d < DP; ++d) sk[ql][part * DP + d] = __float2half_rn(acc[d] * inv_l);
    __syncthreads();
    __half *oh = a.canvas + a.dst_off + (uint64_t)hq * HD * a.pitch;
    for (uint32_t e = tid; e < 32u * HD; e += 128u) { const uint32_t d = e >> 5, c = e & 31u; oh[(uint64_t)d * a.pitch + t0 + c] = sk[c][d]; }
}

// ---- decode attention against a key / value cache ---------------------------------------------------------------------
// Cache layout (both K and V): [h_kv][max_seq][pitch][head_dim] FP16 — the head_dim values of one (head, position, column)
// are contiguous (128 bytes for head_dim 64), so the thread that owns a column reads its key / value row with 16-byte
// loads straight from global memory; no staging, no barrier. One new token per column at position *pos_ptr.

// Rotate q and k in place at the current position and append k and v to the caches: one thread per (head, rotation
// pair, column); the first h_q heads are the query heads, the rest the key heads.
__global__ void __launch_bounds__(256) k44_valu_decode_rope_append_kernel(const AuxArgs a) {
    pdl_enter();
    const uint32_t half = a.head_dim / 2u;
    const uint64_t total = (uint64_t)(a.h_q + a.h_kv) * half * a.pitch;
    const uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    if (i >= total) return;
    const uint32_t col = (uint32_t)(i % a.pitch);
    const uint32_t p = (uint32_t)((i / a.pitch) % half);
    uint32_t h = (uint32_t)(i / ((uint64_t)a.pitch * half));
    const int pos = *a.pos_ptr;
    if (pos < 0 || (uint32_t)pos >= a.max_seq) return;
    const bool is_q = h < a.h_q;
    if (!is_q) h -= a.h_q;
    const uint32_t c0 = h * a.head_dim + p, c1 = c0 + half;
    const uint64_t base = is_q ? a.src_off : a.src2_off;
    __half *r0 = a.canvas + base + (uint64_t)c0 * a.pitch + col, *r1 = a.canvas + base + (uint64_t)c1 * a.pitch + col;
    float s, c;
    sincosf((float)pos * rope_inv_freq(p, a.head_dim, a.neg_log_theta, a.llama3 != 0u), &s, &c);
    const float x0 = __half2float(*r0), x1 = __half2float(*r1);
    const __half y0 = __float2half_rn(x0 * c - x1 * s), y1 = __float2half_rn(x0 * s + x1 * c);
    *r0 = y0; *r1 = y1;
    if (is_q) return;
    const uint64_t row = (((uint64_t)h * a.max_seq + (uint32_t)pos) * a.pitch + col) * a.head_dim;
    a.canvas[a.kcache_off + row + p] = y0;
    a.canvas[a.kcache_off + row + p + half] = y1;
    a.canvas[a.vcache_off + row + p] = a.canvas[a.src3_off + (uint64_t)c0 * a.pitch + col];
    a.canvas[a.vcache_off + row + p + half] = a.canvas[a.src3_off + (uint64_t)c1 * a.pitch + col];
}

// Partial attention of one chunk of kDecodeChunk cache positions. CTA = 128 threads = 16 columns of one key/value head and
// one chunk; 8 lanes share a column, each owning 8 of the 64 dimensions, so that one warp instruction reads the key (or
// value) rows of 4 columns as 512 contiguous bytes. Every lane serves all query heads of the group (the key / value row is
// loaded once for them); dot products are reduced over the 8 lanes by shuffles. UNROLL positions are consumed while the next
// UNROLL are in flight; MINB CTAs per SM bound the register count (four query heads per lane: two positions per batch and 127
// registers keep all 512 CTAs of a 512-position, 64-column step resident at once, 3 % faster per step than four positions
// and 160 registers, which needed a second round of CTAs).
// Output per (chunk, query head, column): 64 unnormalised accumulator values, the running maximum and the sum, FP32,
// [chunk][h_q][pitch][kDecodeRow] (rows of 68 floats: 16-byte aligned for the vector accesses).
template <int G, int UNROLL_, int MINB>
__global__ void __launch_bounds__(128, MINB) k44_valu_decode_attn_partial_kernel(const AuxArgs a, float *partial) {
    pdl_enter();
    constexpr uint32_t HD = 64, UNROLL = UNROLL_;
    const uint32_t cb = blockIdx.x, hkv = blockIdx.y, chunk = blockIdx.z;
    const uint32_t tid = threadIdx.x, j = tid & 7u, col = cb * 16u + (tid >> 3);
    const int pos = *a.pos_ptr;
    const uint32_t p_begin = chunk * kDecodeChunk;
    if (pos < 0 || p_begin > (uint32_t)pos) return;                      // nothing cached in this chunk yet (uniform per CTA)
    const uint32_t p_end = min(p_begin + kDecodeChunk, (uint32_t)pos + 1u);
    const float scale = rsqrtf((float)HD);
    float q[G][8], acc[G][8], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const __half *qh = a.canvas + a.src_off + ((uint64_t)(hkv * G + g) * HD + j * 8u) * a.pitch + col;
#pragma unroll
        for (int e = 0; e < 8; ++e) { q[g][e] = __half2float(qh[(uint64_t)e * a.pitch]) * scale; acc[g][e] = 0.f; }
        m[g] = -65504.0f; l[g] = 0.f;
    }
    const uint64_t row_step = (uint64_t)a.pitch * HD / 8u;                // in 16-byte units
    const uint64_t row0 = (((uint64_t)hkv * a.max_seq + p_begin) * a.pitch + col) * HD / 8u + j;
    const uint4 *const kr = reinterpret_cast<const uint4 *>(a.canvas + a.kcache_off) + row0;
    const uint4 *const vr = reinterpret_cast<const uint4 *>(a.canvas + a.vcache_off) + row0;
    // the rows of the next batch of positions are requested before the current batch is consumed
    uint4 kv[UNROLL], vv[UNROLL], kn[UNROLL], vn[UNROLL];
    auto fetch = [&](uint32_t p, uint4 (&kd)[UNROLL], uint4 (&vd)[UNROLL]) {
#pragma unroll
        for (uint32_t u = 0; u < UNROLL; ++u) {
            const uint32_t pp = min(p + u, p_end - 1u);                  // past the end: re-read the last row (ignored below)
            const uint64_t o = (uint64_t)(pp - p_begin) * row_step;
            kd[u] = __ldg(kr + o);
            vd[u] = __ldg(vr + o);
        }
    };
    fetch(p_begin, kv, vv);
    for (uint32_t p = p_begin; p < p_end; p += UNROLL) {
        if (p + UNROLL < p_end) fetch(p + UNROLL, kn, vn);
#pragma unroll
        for (uint32_t u = 0; u < UNROLL; ++u) {
            if (p + u >= p_end) break;
            float kf[8], vf[8];
            unpack8(kv[u], kf);
            unpack8(vv[u], vf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float dot = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) dot = fmaf(q[g][e], kf[e], dot);
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                dot += __shfl_xor_sync(0xffffffffu, dot, 4);
                const float mn = fmaxf(m[g], dot);
                const float ep = __expf(m[g] - mn), ec = __expf(dot - mn);
                l[g] = l[g] * ep + ec;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(acc[g][e], ep, ec * vf[e]);
                m[g] = mn;
            }
        }
#pragma unroll
        for (uint32_t u = 0; u < UNROLL; ++u) { kv[u] = kn[u]; vv[u] = vn[u]; }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float *out = partial + (((uint64_t)chunk * a.h_q + hkv * G + g) * a.pitch + col) * kDecodeRow;
        *reinterpret_cast<float4 *>(out + j * 8u) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        *reinterpret_cast<float4 *>(out + j * 8u + 4u) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
        if (j == 0u) { out[HD] = m[g]; out[HD + 1u] = l[g]; }
    }
}

// combine the chunks: 8 lanes per (query head, column), 8 dimensions each
__global__ void __launch_bounds__(256) k44_valu_decode_attn_combine_kernel(const AuxArgs a, const float *partial) {
    pdl_enter();
    constexpr uint32_t HD = 64;
    const uint64_t total = (uint64_t)a.h_q * a.pitch * 8u;
    const uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    if (i >= total) return;
    const uint32_t j = (uint32_t)(i & 7u), col = (uint32_t)((i >> 3) % a.pitch), hq = (uint32_t)((i >> 3) / a.pitch);
    const int pos = *a.pos_ptr;
    if (pos < 0) return;
    const uint32_t chunks = (uint32_t)pos / kDecodeChunk + 1u;
    const uint64_t stride = (uint64_t)a.h_q * a.pitch * kDecodeRow;
    const float *pc = partial + ((uint64_t)hq * a.pitch + col) * kDecodeRow;
    // all loads of a batch of 8 chunks are issued before any is used (the chunks are far apart in memory)
    float M = -65504.0f;
    for (uint32_t c0 = 0; c0 < chunks; c0 += 8u) {
        float mv[8];
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) mv[u] = pc[(uint64_t)min(c0 + u, chunks - 1u) * stride + HD];
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) M = fmaxf(M, mv[u]);
    }
    float L = 0.f, o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (uint32_t c0 = 0; c0 < chunks; c0 += 8u) {
        float mv[8], lv[8];
        float4 x[8], y[8];
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) {
            const float *r = pc + (uint64_t)min(c0 + u, chunks - 1u) * stride;
            mv[u] = r[HD]; lv[u] = r[HD + 1u];
            x[u] = *reinterpret_cast<const float4 *>(r + j * 8u);
            y[u] = *reinterpret_cast<const float4 *>(r + j * 8u + 4u);
        }
#pragma unroll
        for (uint32_t u = 0; u < 8u; ++u) {
            if (c0 + u >= chunks) break;
            const float w = __expf(mv[u] - M);
            L = fmaf(lv[u], w, L);
            o[0] = fmaf(x[u].x, w, o[0]); o[1] = fmaf(x[u].y, w, o[1]); o[2] = fmaf(x[u].z, w, o[2]); o[3] = fmaf(x[u].w, w, o[3]);
            o[4] = fmaf(y[u].x, w, o[4]); o[5] = fmaf(y[u].y, w, o[5]); o[6] = fmaf(y[u].z, w, o[6]); o[7] = fmaf(y[u].w, w, o[7]);
        }
    }
    const float inv = 1.0f / L;
    __half *dst = a.canvas + a.dst_off + ((uint64_t)hq * HD + j * 8u) * a.pitch + col;
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[(uint64_t)e * a.pitch] = __float2half_rn(o[e] * inv);
}
// ---- token I/O ---------------------------------------------------------------------------------------------------------
// Embedding gather: column b of the destination tensor becomes row tokens[b] of the table. One thread per (8 channels,
// column): one 16-byte load from the table row, eight 2-byte stores (consecutive lanes = consecutive columns).
__global__ void __launch_bounds__(256) k44_valu_embed_kernel(const AuxArgs a) {
    pdl_enter();
    const uint32_t chunks = a.rows / 8u;
    const uint64_t i = (uint64_t)blockIdx.x * 256u + threadIdx.x;
    if (i >= (uint64_t)chunks * a.pitch) return;
    const uint32_t col = (uint32_t)(i % a.pitch), c8 = (uint32_t)(i / a.pitch);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (col < a.columns) {
        const int tok = a.tokens[col];
        if (tok >= 0 && (uint32_t)tok < a.vocab) v = *reinterpret_cast<const uint4 *>(a.table + (uint64_t)tok * a.rows + c8 * 8u);
    }
    const __half *h = reinterpret_cast<const __half *>(&v);
    __half *dst = a.canvas + a.dst_off + (uint64_t)c8 * 8u * a.pitch + col;
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[(uint64_t)e * a.pitch] = h[e];
}

// Arg-max over the rows of a tensor, per column. FP16 values are mapped to integer keys that sort like the numbers; a key
// and the complement of its row are packed into 64 bits so that one max() picks the largest value and, among equals, the
// lowest row. NaN sorts below everything.
__device__ __forceinline__ unsigned long long argmax_pack(__half v, uint32_t row) {
    const uint16_t u = __half_as_ushort(v);
    uint32_t key = (u & 0x8000u) ? (uint32_t)(0x7fffu - (u & 0x7fffu)) : (uint32_t)(0x8000u + u);
    if ((u & 0x7fffu) > 0x7c00u) key = 0u;
    return ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - row);
}

// stage 1: CTA = kArgmaxChunk rows x 64 columns; 4 threads per column take every fourth row
__global__ void __launch_bounds__(256) k44_valu_argmax_partial_kernel(const AuxArgs a) {
    pdl_enter();
    __shared__ unsigned long long best_s[4][64];
    const uint32_t col = blockIdx.x * 64u + (threadIdx.x & 63u), ph = threadIdx.x >> 6;
    const uint32_t r0 = blockIdx.y * kArgmaxChunk, r1 = min(a.rows, r0 + kArgmaxChunk);
    unsigned long long best = 0ull;
    const __half *src = a.canvas + a.src_off + col;
    for (uint32_t r = r0 + ph; r < r1; r += 4u) best = max(best, argmax_pack(src[(uint64_t)r * a.pitch], r));
    best_s[ph][threadIdx.x & 63u] = best;
    __syncthreads();
    if (ph == 0u) {
        const uint32_t c = threadIdx.x & 63u;
        best = max(max(best_s[0][c], best_s[1][c]), max(best_s[2][c], best_s[3][c]));
        a.argmax_scratch[(uint64_t)blockIdx.y * a.pitch + col] = best;
    }
}

// stage 2: one thread per column folds the chunks, writes the winning row and optionally feeds it back
__global__ void __launch_bounds__(256) k44_valu_argmax_final_kernel(const AuxArgs a) {
    pdl_enter();
    const uint32_t col = blockIdx.x * 256u + threadIdx.x;
    const uint32_t chunks = (a.rows + kArgmaxChunk - 1u) / kArgmaxChunk;
    if (col < a.pitch) {
        unsigned long long best = 0ull;
        for (uint32_t c0 = 0; c0 < chunks; c0 += 8u) {
            unsigned long long v[8];
#pragma unroll
            for (uint32_t u = 0; u < 8u; ++u) v[u] = a.argmax_scratch[(uint64_t)min(c0 + u, chunks - 1u) * a.pitch + col];
#pragma unroll
            for (uint32_t u = 0; u < 8u; ++u) best = max(best, v[u]);
        }
        const int row = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
        a.next_tokens[col] = row;
        if (a.advance && col < a.columns) a.tokens[col] = row;
    }
    if (a.advance && col == 0u && a.pos_rw) {
        const int p = *a.pos_rw;
        *a.pos_rw = (a.max_seq && p + 1 >= (int)a.max_seq) ? (int)a.max_seq - 1 : p + 1;
    }
}

cudaError_t launch_aux(const AuxArgs &a, bool pdl, cudaStream_t s) {
    cudaError_t e = cudaSuccess;
    switch (a.kind) {
    case AUX_RMSNORM: {
        if (a.pitch % 8u || a.rows == 0) return cudaErrorInvalidValue;
        const dim3 grid(a.pitch / 8u), block(1024);
        if (a.rows <= 2048u) e = launch_k(k44_valu_rmsnorm_kernel<2>, grid, block, pdl, s, a);
        else if (a.rows <= 4096u) e = launch_k(k44_valu_rmsnorm_kernel<4>, grid, block, pdl, s, a);
        else e = launch_k(k44_valu_rmsnorm_kernel<0>, grid, block, pdl, s, a);
        break;
    }
    case AUX_SWIGLU: {
        const uint64_t n8 = (uint64_t)a.rows * a.pitch / 8u;
        const uint32_t grid = (uint32_t)std::min<uint64_t>((n8 + 255u) / 256u, 148u * 16u);
        e = launch_k(k44_valu_swiglu_kernel, dim3(grid ? grid : 1u), dim3(256), pdl, s, a);
        break;
    }
    case AUX_ROPE_ATTN: {
        if (a.head_dim != 64u && a.head_dim != 128u) return cudaErrorInvalidValue;
        if (a.pitch % 32u || a.seq_len % 32u || a.h_kv == 0 || a.h_q % a.h_kv) return cudaErrorInvalidValue;
        const uint32_t groups = a.pitch / 8u, half = a.head_dim / 2u;
        e = launch_k(k44_valu_rope_kernel, dim3((uint32_t)(((uint64_t)a.h_q * half * groups + 255u) / 256u)), dim3(256), pdl, s, a, a.src_off, a.h_q);
        if (e == cudaSuccess) e = launch_k(k44_valu_rope_kernel, dim3((uint32_t)(((uint64_t)a.h_kv * half * groups + 255u) / 256u)), dim3(256), pdl, s, a, a.src2_off, a.h_kv);
        const dim3 grid((a.columns + 31u) / 32u, a.h_q);
        if (e == cudaSuccess) e = a.head_dim == 64u ? launch_k(k44_valu_causal_attn_kernel<64>, grid, dim3(128), pdl, s, a)
                                                    : launch_k(k44_valu_causal_attn_kernel<128>, grid, dim3(128), pdl, s, a);
        break;
    }
    case AUX_DECODE_ATTN: {
        // rotary on q and k at the current position + cache append of k / v, partial attention per chunk, combine
        if (a.head_dim != 64u || a.pitch % 32u || !a.pos_ptr || !a.partial || a.h_kv == 0 || a.h_q % a.h_kv) return cudaErrorInvalidValue;
        e = launch_k(k44_valu_decode_rope_append_kernel, dim3((uint32_t)(((uint64_t)(a.h_q + a.h_kv) * (a.head_dim / 2u) * a.pitch + 255u) / 256u)), dim3(256), pdl, s, a);
        const dim3 grid(a.pitch / 16u, a.h_kv, (a.max_seq + kDecodeChunk - 1u) / kDecodeChunk);
        if (e != cudaSuccess) break;
        switch (a.h_q / a.h_kv) {
        case 1: e = launch_k(k44_valu_decode_attn_partial_kernel<1, 4, 4>, grid, dim3(128), pdl, s, a, a.partial); break;
        case 2: e = launch_k(k44_valu_decode_attn_partial_kernel<2, 4, 4>, grid, dim3(128), pdl, s, a, a.partial); break;
        case 4: e = launch_k(k44_valu_decode_attn_partial_kernel<4, 2, 4>, grid, dim3(128), pdl, s, a, a.partial); break;
        case 8: e = launch_k(k44_valu_decode_attn_partial_kernel<8, 4, 2>, grid, dim3(128), pdl, s, a, a.partial); break;
        default: return cudaErrorInvalidValue;
        }
        if (e == cudaSuccess)
            e = launch_k(k44_valu_decode_attn_combine_kernel, dim3((uint32_t)(((uint64_t)a.h_q * a.pitch * 8u + 255u) / 256u)), dim3(256), pdl, s, a, (const float *)a.partial);
        break;
    }
    case AUX_EMBED:
        if (a.rows % 8u || !a.table || !a.tokens) return cudaErrorInvalidValue;
        e = launch_k(k44_valu_embed_kernel, dim3((uint32_t)(((uint64_t)(a.rows / 8u) * a.pitch + 255u) / 256u)), dim3(256), pdl, s, a);
        break;
    case AUX_ARGMAX: {
        if (a.pitch % 64u || !a.argmax_scratch || !a.next_tokens || a.rows == 0) return cudaErrorInvalidValue;
        e = launch_k(k44_valu_argmax_partial_kernel, dim3(a.pitch / 64u, (a.rows + kArgmaxChunk - 1u) / kArgmaxChunk), dim3(256), pdl, s, a);
        if (e == cudaSuccess) e = launch_k(k44_valu_argmax_final_kernel, dim3((a.pitch + 255u) / 256u), dim3(256), pdl, s, a);
        break;
    }
    case AUX_MAXPOOL2: case AUX_MAXPOOL5: case AUX_UPSAMPLE2: case AUX_S2D: case AUX_UPCONV_SCATTER: case AUX_HALO_CLEAR:
        e = launch_image_aux(a, s);
        break;
    default: return cudaErrorInvalidValue;
    }
    return e;
}

}  // namespace k44b
