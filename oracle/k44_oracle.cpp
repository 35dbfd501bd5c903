// k44_oracle.cpp — TEST INFRASTRUCTURE ONLY. CPU restatement of the SNNtome wave-executor maths.
//
// This file is the checker that the CUDA path is compared against. It is never linked into, imported
// by or called from the shipped library; only the test-suite, the smoke check and the benchmark's
// CPU-baseline leg load it.
//
// PARITY UNPINNED for output values: the reference ships no golden vectors, no fixtures and no CPU
// executor for this path, and its licence forbids compiling or running it. What *is* pinned:
//   * FNV-1a-64 against the published known-answer vectors (tests/test_oracle.py),
//   * FP16 conversion against numpy.float16 for all 65536 bit patterns and random floats,
//   * the wave arithmetic against a numpy float64 restatement and numpy.matmul in the dense case.
//
// Each function cites the reference location whose behaviour it restates (paths relative to the
// reference project root). Nothing here was copied; the arithmetic is written from the formulas.
//
// Build: see oracle/Makefile (g++ -O3 -march=native -fopenmp -shared -fPIC).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- FP16 <-> FP32, round to nearest even, subnormals kept, overflow -> inf --------------------
// Behaviour described by wavec/k44_plan_types.hpp:21-87; written independently around the
// "scale into the target grid and let the FPU round" idea instead of manual mantissa surgery.
inline uint16_t f32_to_f16_rte(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t absu = u & 0x7fffffffu;
    if (absu >= 0x7f800000u) {                       // inf / nan
        if (absu == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
        // the reference keeps the top mantissa bits and forces the payload non-zero
        return (uint16_t)(sign | 0x7c00u | ((absu & 0x007fffffu) >> 13) | 1u);
    }
    if (absu >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);   // >= 65520 rounds to inf
    if (absu < 0x38800000u) {                        // below the smallest normal half: subnormal grid
        // the half subnormal grid has spacing 2^-24: round |f| * 2^24 to an integer, RTE.
        float a;
        std::memcpy(&a, &absu, 4);
        const float scaled = a * 16777216.0f;        // exact (power of two), <= 1024
        const float r = std::nearbyintf(scaled);     // default rounding mode = RTE
        return (uint16_t)(sign | (uint32_t)r);       // r == 1024 lands on the smallest normal: correct
    }
    // normal range: add half an ulp of the 10-bit mantissa (plus the tie-to-even correction)
    const uint32_t lsb = (absu >> 13) & 1u;
    const uint32_t rounded = absu + 0x0fffu + lsb;
    return (uint16_t)(sign | ((rounded - 0x38000000u) >> 13));
}

// Double -> half with ONE rounding (round to nearest, ties to even): the value is first rounded onto the half grid
// in double arithmetic (spacing 2^(e-10) for a normal result, 2^-24 below 2^-14; division and product by a power of
// two are exact, nearbyint uses the default rounding mode), then the exactly representable result is encoded.
// Rounding through float first would round twice (a value a hair above a half-way point of the half grid can
// land exactly on it as a float).
inline uint16_t f64_to_f16_rte(double v) {
    if (std::isnan(v)) return 0x7e00u;
    const double a = std::fabs(v);
    if (a >= 65520.0) return (uint16_t)((std::signbit(v) ? 0x8000u : 0u) | 0x7c00u);
    int e = 0;
    (void)std::frexp(a, &e);                          // a = m * 2^e, 0.5 <= m < 1  ->  a in [2^(e-1), 2^e)
    const int spacing_exp = (a < 6.103515625e-05) ? -24 : (e - 1) - 10;
    const double r = std::ldexp(std::nearbyint(std::ldexp(a, -spacing_exp)), spacing_exp);
    return f32_to_f16_rte((float)(std::signbit(v) ? -r : r));   // exact: r is on the half grid
}

inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t em = h & 0x7fffu;
    uint32_t u;
    if (em >= 0x7c00u) {
        u = sign | 0x7f800000u | ((em & 0x3ffu) << 13);
    } else if (em >= 0x0400u) {
        u = sign | ((em << 13) + 0x38000000u);
    } else {
        const float v = (float)em * (1.0f / 16777216.0f);   // exact
        std::memcpy(&u, &v, 4);
        u |= sign;
    }
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// Activation set of kernels/cuda/kernel44_cuda_pack.cuh:54-58 evaluated in double, plus value 5
// (exact erf GELU) which the reference does not have.
inline double activate(double v, int act) {
    switch (act) {
    case 1: return v > 0.0 ? v : 0.0;
    case 2: return 1.0 / (1.0 + std::exp(-v));
    case 3: return v / (1.0 + std::exp(-v));
    case 4: return v > 0.1 * v ? v : 0.1 * v;
    case 5: return 0.5 * v * (1.0 + std::erf(v * 0.70710678118654752440));
    default: return v;
    }
}

}  // namespace

extern "C" {

// FNV-1a 64-bit — wavec/k44_tcff_io.hpp:10-17 (standard offset basis and prime).
uint64_t k44o_fnv1a64(const uint8_t *data, uint64_t len) {
    uint64_t h = 14695981039346656037ull;
    for (uint64_t i = 0; i < len; ++i) {
        h = (h ^ data[i]) * 1099511628211ull;
    }
    return h;
}

void k44o_f32_to_f16(const float *src, uint16_t *dst, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = f32_to_f16_rte(src[i]);
}

void k44o_f64_to_f16(const double *src, uint16_t *dst, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = f64_to_f16_rte(src[i]);
}

void k44o_f16_to_f32(const uint16_t *src, float *dst, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = f16_to_f32(src[i]);
}

// Row-major [cout][B] <-> the file's 16x16 tile order — wavec/k44_plan_types.hpp:363-394.
// A weight row is cut into 8-half (16-byte) vectors. Tiles are 16 neurons x 16 synapses, walked
// neuron-block major; inside a tile the 32 vectors are ordered (k_half, neuron): vector v holds
// neuron (v & 15), synapse half (v >> 4).
void k44o_rowmajor_to_wmma(const uint16_t *row_major, uint16_t *wmma, uint32_t cout, uint32_t B) {
    const uint32_t kt = B / 16;
    for (uint32_t nb = 0; nb < cout / 16; ++nb)
        for (uint32_t kb = 0; kb < kt; ++kb)
            for (uint32_t v = 0; v < 32; ++v) {
                const uint32_t neuron = nb * 16 + (v & 15);
                const uint32_t k0 = kb * 16 + (v >> 4) * 8;
                std::memcpy(wmma + (((uint64_t)nb * kt + kb) * 32 + v) * 8,
                            row_major + (uint64_t)neuron * B + k0, 16);
            }
}

void k44o_wmma_to_rowmajor(const uint16_t *wmma, uint16_t *row_major, uint32_t cout, uint32_t B) {
    const uint32_t kt = B / 16;
    for (uint32_t nb = 0; nb < cout / 16; ++nb)
        for (uint32_t kb = 0; kb < kt; ++kb)
            for (uint32_t v = 0; v < 32; ++v) {
                const uint32_t neuron = nb * 16 + (v & 15);
                const uint32_t k0 = kb * 16 + (v >> 4) * 8;
                std::memcpy(row_major + (uint64_t)neuron * B + k0,
                            wmma + (((uint64_t)nb * kt + kb) * 32 + v) * 8, 16);
            }
}

// One wave over a 1-D token layout, in place on the canvas.
//
//   Y[y_off + tile_off_Y[t] + out_j*pitch + c] =
//       f16_rte( epilogue( bias[j] + sum_s W[j][s] * X[x_base + tile_off_X[t] + idx[j/G][s] + c] ) )
//
// Semantics: kernels/cuda/kernel44_cuda_pack.cuh:190-216 (addressing, bias-initialised accumulator),
// :69-126 (epilogue: residual added BEFORE the activation when a cout map is present, AFTER it
// otherwise; optional uint16 output-row remap), wavec/k44_plan_types.hpp:498-516 (64-column tiles).
// Operands are the FP16-quantised values; accumulation is in double ("stage 2" of
// whitepaper/sparse_wmma_kernel/tests/error_collapse_test.cpp:297-347), so the only rounding is
// the final store. Padded synapse slots are consumed as stored (index 0, weight 0), exactly like
// the reference kernels do.
//
// Token shift (the receptive-field variant; the reference expresses a shifted tap as an element-granular
// offset, kernels/cuda/kernel44_cuda_pack.cuh:153-159, wavec/k44_plan_types.hpp:592-600): when `shifts` is given,
// synapse s of group g reads its row `shifts[g*B+s]` columns earlier, and — causal padding, which the flat
// offsets of the reference cannot express — columns whose position inside their frame of `frame_len` columns
// is smaller than the shift read zero instead of the previous frame's tail (frame_len 0: one frame per row).
//
// rows_begin/rows_end restrict the neurons computed (sampled checks on very large waves).
// Returns 0, or -1 if an index would leave the canvas (nothing is written in that case).
int k44o_wave_forward(uint16_t *canvas, uint64_t canvas_elems, const uint16_t *w_row_major,
                      const uint32_t *idx, const uint16_t *bias, const uint16_t *cout_map,
                      uint32_t cout, uint32_t group, uint32_t B, int act, int has_residual,
                      uint64_t y_off, uint64_t res_off, uint64_t x_base_off, uint32_t pitch,
                      const uint32_t *tile_off_x, const uint32_t *tile_off_y, uint32_t num_tiles,
                      uint32_t rows_begin, uint32_t rows_end, const uint8_t *shifts, uint32_t frame_len) {
    if (rows_end > cout) rows_end = cout;
    // bounds check first: every read and write must stay inside the canvas
    uint32_t max_idx = 0;
    for (uint64_t i = (uint64_t)(rows_begin / group) * B; i < (uint64_t)((rows_end + group - 1) / group) * B; ++i)
        if (idx[i] > max_idx) max_idx = idx[i];
    for (uint32_t t = 0; t < num_tiles; ++t) {
        if (x_base_off + tile_off_x[t] + max_idx + 64 > canvas_elems) return -1;
    }
    for (uint32_t j = rows_begin; j < rows_end; ++j) {
        const uint64_t out_j = cout_map ? cout_map[j] : j;
        for (uint32_t t = 0; t < num_tiles; ++t) {
            if (y_off + tile_off_y[t] + out_j * pitch + 64 > canvas_elems) return -1;
            if (has_residual && res_off + tile_off_y[t] + out_j * pitch + 64 > canvas_elems) return -1;
        }
    }
    // All reads come from earlier waves' regions, all writes go to this wave's region; a snapshot
    // of the outputs is staged so that a plan that (incorrectly) aliases them still behaves like
    // the GPU's "read old data" order as far as possible. Writes are applied at the end.
    const int64_t nrows = (int64_t)rows_end - (int64_t)rows_begin;
    std::vector<uint16_t> out((size_t)(nrows > 0 ? nrows : 0) * num_tiles * 64);
#pragma omp parallel
    {
        std::vector<double> wrow(B);
        std::vector<double> acc(64);
#pragma omp for schedule(dynamic, 4)
        for (int64_t jj = 0; jj < nrows; ++jj) {
            const uint32_t j = rows_begin + (uint32_t)jj;
            const uint32_t *irow = idx + (uint64_t)(j / group) * B;
            for (uint32_t s = 0; s < B; ++s) wrow[s] = (double)f16_to_f32(w_row_major[(uint64_t)j * B + s]);
            const double b = bias ? (double)f16_to_f32(bias[j]) : 0.0;
            const uint64_t out_j = cout_map ? cout_map[j] : j;
            for (uint32_t t = 0; t < num_tiles; ++t) {
                for (int c = 0; c < 64; ++c) acc[c] = b;
                const uint16_t *xt = canvas + x_base_off + tile_off_x[t];
                for (uint32_t s = 0; s < B; ++s) {
                    const double w = wrow[s];
                    const uint16_t *xr = xt + irow[s];
                    if (!shifts) {
                        for (int c = 0; c < 64; ++c) acc[c] += w * (double)f16_to_f32(xr[c]);
                    } else {
                        const uint32_t sh = shifts[(uint64_t)(j / group) * B + s];
                        const uint32_t flen = frame_len ? frame_len : pitch;
                        for (int c = 0; c < 64; ++c) {
                            const uint32_t col = tile_off_x[t] % pitch + (uint32_t)c;     // column inside the row
                            if (col % flen >= sh) acc[c] += w * (double)f16_to_f32(xr[(int64_t)c - (int64_t)sh]);
                        }
                    }
                }
                const uint16_t *rr = has_residual ? canvas + res_off + tile_off_y[t] + out_j * pitch : nullptr;
                uint16_t *o = out.data() + ((size_t)jj * num_tiles + t) * 64;
                for (int c = 0; c < 64; ++c) {
                    double v = acc[c];
                    const double r = rr ? (double)f16_to_f32(rr[c]) : 0.0;
                    if (rr && cout_map) v += r;
                    v = activate(v, act);
                    if (rr && !cout_map) v += r;
                    o[c] = f64_to_f16_rte(v);
                }
            }
        }
    }
    for (int64_t jj = 0; jj < nrows; ++jj) {
        const uint32_t j = rows_begin + (uint32_t)jj;
        const uint64_t out_j = cout_map ? cout_map[j] : j;
        for (uint32_t t = 0; t < num_tiles; ++t)
            std::memcpy(canvas + y_off + tile_off_y[t] + out_j * pitch,
                        out.data() + ((size_t)jj * num_tiles + t) * 64, 128);
    }
    return 0;
}

// One wave over 2-D image planes (wavec/k44_plan_types.hpp:517-569, kernels/cuda/kernel44_cuda_pack.cuh:116-124, 190-216):
// tile t gathers 64 consecutive elements from x_base + tile_off_x[t] + idx[j/G][s] and stores 64 results at
// y_off + j * plane_stride + tile offset, where the tile offset is tile_off_y[t], or — masked layouts — 4 * (tile_off_y[t] &
// 0xffff) with only those 4-element quads q written whose bit 16 + q of tile_off_y[t] is set. Residual after the activation
// (image waves carry no row map). Double accumulation, one rounding. Returns -1 if anything would leave the canvas.
int k44o_wave_forward_2d(uint16_t *canvas, uint64_t canvas_elems, const uint16_t *w_row_major, const uint32_t *idx, const uint16_t *bias,
                         uint32_t cout, uint32_t group, uint32_t B, int act, int has_residual, uint64_t y_off, uint64_t res_off,
                         uint64_t x_base_off, uint32_t plane_stride, const uint32_t *tile_off_x, const uint32_t *tile_off_y, uint32_t num_tiles,
                         int tile_mask) {
    uint32_t max_idx = 0;
    for (uint64_t i = 0; i < (uint64_t)(cout / group) * B; ++i) max_idx = idx[i] > max_idx ? idx[i] : max_idx;
    auto y_of = [&](uint32_t t) -> uint64_t { return tile_mask ? (uint64_t)(tile_off_y[t] & 0xffffu) << 2 : tile_off_y[t]; };
    for (uint32_t t = 0; t < num_tiles; ++t) {
        if (x_base_off + tile_off_x[t] + max_idx + 64 > canvas_elems) return -1;
        if (y_off + (uint64_t)(cout - 1) * plane_stride + y_of(t) + 64 > canvas_elems) return -1;
        if (has_residual && res_off + (uint64_t)(cout - 1) * plane_stride + y_of(t) + 64 > canvas_elems) return -1;
    }
    std::vector<uint16_t> out((size_t)cout * num_tiles * 64);
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t j = 0; j < (int64_t)cout; ++j) {
        const uint32_t *irow = idx + (uint64_t)(j / group) * B;
        const double b = bias ? (double)f16_to_f32(bias[j]) : 0.0;
        for (uint32_t t = 0; t < num_tiles; ++t) {
            double acc[64];
            for (int c = 0; c < 64; ++c) acc[c] = b;
            const uint16_t *xt = canvas + x_base_off + tile_off_x[t];
            for (uint32_t s = 0; s < B; ++s) {
                const double w = (double)f16_to_f32(w_row_major[(uint64_t)j * B + s]);
                const uint16_t *xr = xt + irow[s];
                for (int c = 0; c < 64; ++c) acc[c] += w * (double)f16_to_f32(xr[c]);
            }
            const uint16_t *rr = has_residual ? canvas + res_off + (uint64_t)j * plane_stride + y_of(t) : nullptr;
            uint16_t *o = out.data() + ((size_t)j * num_tiles + t) * 64;
            for (int c = 0; c < 64; ++c) {
                double v = activate(acc[c], act);
                if (rr) v += (double)f16_to_f32(rr[c]);
                o[c] = f64_to_f16_rte(v);
            }
        }
    }
    for (uint32_t j = 0; j < cout; ++j)
        for (uint32_t t = 0; t < num_tiles; ++t) {
            uint16_t *dst = canvas + y_off + (uint64_t)j * plane_stride + y_of(t);
            const uint16_t *src = out.data() + ((size_t)j * num_tiles + t) * 64;
            const uint32_t mask = tile_mask ? tile_off_y[t] >> 16 : 0xffffu;
            for (uint32_t q = 0; q < 16; ++q)
                if ((mask >> q) & 1u) std::memcpy(dst + 4 * q, src + 4 * q, 8);
        }
    return 0;
}

// Same arithmetic but with FP32 accumulation in 16-synapse chunks followed by the FP16 store —
// "stage 3" of whitepaper/sparse_wmma_kernel/tests/error_collapse_test.cpp:297-347. Used only for
// the sanity band on expected GPU-vs-exact error, never as the parity reference.
void k44o_dot_stage3(const uint16_t *w, const uint16_t *x, uint32_t B, float bias, float *out) {
    float acc = bias;
    for (uint32_t s0 = 0; s0 < B; s0 += 16) {
        float part = 0.0f;
        for (uint32_t s = s0; s < s0 + 16 && s < B; ++s) part += f16_to_f32(w[s]) * f16_to_f32(x[s]);
        acc += part;
    }
    *out = f16_to_f32(f32_to_f16_rte(acc));
}

int k44o_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void k44o_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
