// Host-side plan model of the wave executor: FP16 helpers, padding rules, the 1-D token layout,
// wave / plan structs and the 16x16-tile weight order used by the .tcff container.
//
// Field meaning mirrors the reference structs so that a maintainer can map one onto the other:
//   HostWave  <-> K44ExecCmd   (wavec/k44_plan_types.hpp:603-650)
//   HostPlan  <-> K44WavePlan  (wavec/k44_plan_types.hpp:663-693)
//   Layout1D  <-> K44ResDesc, 1-D branch (wavec/k44_plan_types.hpp:498-516, 576-600)
// The code is written fresh against those semantics.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace k44b {

// ---- FP16 / BF16 ------------------------------------------------------------------------------
// float -> half, round to nearest even, subnormals preserved, overflow to inf, NaN kept NaN
// (behaviour of wavec/k44_plan_types.hpp:21-60). Implemented with integer rounding on the bit
// pattern: a "magic" right shift that carries naturally from mantissa into exponent.
inline uint16_t float_to_half(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7fffffffu;
    if (x > 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((x & 0x007fffffu) >> 13) | 1u);
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (x < 0x33000001u) return sign;                 // <= 2^-25 rounds to zero (tie goes to even)
    uint32_t shift, mant;
    if (x < 0x38800000u) {                            // result is subnormal
        const uint32_t e = x >> 23;                   // biased float exponent, 102..112
        mant = (x & 0x007fffffu) | 0x00800000u;
        shift = 126u - e;                             // 14..24 bits dropped
        const uint32_t kept = mant >> shift;
        const uint32_t rem = mant & ((1u << shift) - 1u);
        const uint32_t half = 1u << (shift - 1u);
        return (uint16_t)(sign | (kept + ((rem > half) || (rem == half && (kept & 1u)))));
    }
    const uint32_t rebias = x - 0x38000000u;          // exponent now half-biased, 13 extra mantissa bits
    const uint32_t kept = rebias >> 13;
    const uint32_t rem = rebias & 0x1fffu;
    return (uint16_t)(sign | (kept + ((rem > 0x1000u) || (rem == 0x1000u && (kept & 1u)))));
}

inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t em = h & 0x7fffu, out;
    if (em >= 0x7c00u) {
        out = sign | 0x7f800000u | ((em & 0x3ffu) << 13);
    } else if (em >= 0x0400u) {
        out = sign | ((em << 13) + 0x38000000u);
    } else if (em == 0) {
        out = sign;
    } else {
        int e = 113;                                  // normalise the subnormal
        while (!(em & 0x0400u)) { em <<= 1; --e; }
        out = sign | ((uint32_t)e << 23) | ((em & 0x3ffu) << 13);
    }
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}

inline float bf16_to_float(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// ---- padding rules (wavec/k44_plan_types.hpp:157-186) ------------------------------------------
inline uint32_t pad_cout(uint32_t v) { return std::max(16u, (v + 15u) & ~15u); }
inline uint32_t pad_fan_in(uint32_t v) { return std::max(64u, (v + 31u) & ~31u); }

inline uint32_t choose_group_size(uint32_t cout_pad, uint32_t num_tiles, uint32_t forced) {
    for (uint32_t g = forced; g >= 16u; g >>= 1)
        if (cout_pad % g == 0u) return g;
    if (cout_pad % 128u == 0u && (cout_pad >= 640u || num_tiles <= 64u)) return 128u;
    if (cout_pad % 64u == 0u) return 64u;
    if (cout_pad % 32u == 0u) return 32u;
    return 16u;
}

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_SIGMOID = 2, ACT_SILU = 3, ACT_LEAKY_RELU = 4, ACT_GELU = 5 };

inline const char *act_name(int a) {
    static const char *names[] = {"NONE", "RELU", "SIGMOID", "SILU", "LEAKY_RELU", "GELU"};
    return (a >= 0 && a <= 5) ? names[a] : "NONE";
}

// ---- 1-D token layout ---------------------------------------------------------------------------
// A tensor [C][1][W] lives in C canvas rows of `channel_stride` FP16 elements; columns are cut into
// 64-wide tiles; tile t of frame f starts at f*single_stride + 64*t.
struct Layout1D {
    uint32_t width = 0;            // valid columns (tokens)
    uint32_t frames = 1;
    uint32_t tiles_per_frame = 0;
    uint32_t single_stride = 0;
    uint32_t channel_stride = 0;   // "pitch"
    uint32_t num_tiles = 0;

    void init(uint32_t w, uint32_t nframes = 1) {
        width = w;
        frames = std::max(1u, nframes);
        tiles_per_frame = (w + 63u) / 64u;
        single_stride = tiles_per_frame * 64u;
        channel_stride = frames * single_stride;
        num_tiles = frames * tiles_per_frame;
    }
    uint64_t offset(uint32_t ch, uint32_t x, uint32_t frame = 0) const {
        return (uint64_t)ch * channel_stride + (uint64_t)frame * single_stride + x;
    }
};

// ---- 2-D image layout (wavec/k44_plan_types.hpp:517-569, 576-600) ---------------------------------
// A tensor [C][H][W] lives in C planes of `channel_stride` FP16 elements; a plane is the image with a zero halo around it
// (one row above and below, four elements left of every row) so that the taps of a 3x3 convolution never need a bounds
// check. Waves still work on tiles of 64 consecutive elements of a plane:
//   * W a multiple of 64 ("aligned"): rows of W + 8 elements (4 halo + W + 4 halo), a tile is 64 pixels of one image row.
//     tile_off_x is anchored one row up and one element left of the tile (so every tap offset is non-negative),
//     tile_off_y at the tile's first pixel;
//   * otherwise ("masked"): rows of W + 4 elements, tiles run on across the rows (the next row's left halo doubles as the
//     right halo) and would overwrite halo elements, so every tile carries a 16-bit mask — bit q set iff the four elements
//     4q .. 4q+3 of the tile are pixels (W is a multiple of 4) — packed into tile_off_y as
//     (plane offset of the tile / 4) & 0xffff | mask << 16; such planes hold at most 2^18 elements.
// Several frames per wave (wavec_set_batch_size): the frames of one channel lie one after the other, `single_stride` apart
// (channel_stride = frames * single_stride, wavec/k44_plan_types.hpp:498-516), and the tile tables list every frame's tiles.
struct Layout2D {
    uint32_t H = 0, W = 0, H_pad = 0, W_pad = 0;
    uint32_t tiles_per_frame = 0, num_tiles = 0;
    uint32_t single_stride = 0, channel_stride = 0;
    bool masked = false;
    std::vector<uint32_t> tile_off_x, tile_off_y;

    uint32_t frames = 1;

    bool init(uint32_t h, uint32_t w, uint32_t nframes = 1) {
        H = h; W = w; frames = nframes ? nframes : 1u;
        tile_off_x.clear(); tile_off_y.clear();
        if (h == 0 || w == 0 || w % 4u) return false;
        H_pad = H + 2u;
        if (W % 64u == 0u) {
            masked = false;
            W_pad = W + 8u;
            single_stride = H_pad * W_pad;
            const uint32_t per_row = W / 64u;
            tiles_per_frame = H * per_row;
            for (uint32_t ty = 0; ty < H; ++ty)
                for (uint32_t tx = 0; tx < per_row; ++tx) {
                    tile_off_x.push_back(ty * W_pad + (4u + tx * 64u - 1u));
                    tile_off_y.push_back((ty + 1u) * W_pad + (4u + tx * 64u));
                }
        } else {
            masked = true;
            W_pad = W + 4u;
            tiles_per_frame = (H * W_pad + 63u) / 64u;
            single_stride = (2u * W_pad + tiles_per_frame * 64u + 63u) & ~63u;
            if ((uint64_t)single_stride * frames > (1u << 18)) return false;   // the packed tile offset has 16 bits of quads
            for (uint32_t t = 0; t < tiles_per_frame; ++t) {
                const uint32_t y1 = W_pad + 4u + t * 64u;
                tile_off_x.push_back(y1 - W_pad - 1u);
                uint32_t mask = 0;
                for (uint32_t q = 0; q < 16u; ++q) {
                    const uint32_t rel = t * 64u + q * 4u;
                    if (rel / W_pad < H && rel % W_pad < W) mask |= 1u << q;
                }
                tile_off_y.push_back(((y1 >> 2) & 0xffffu) | (mask << 16));
            }
        }
        if ((uint64_t)single_stride * frames > 0x7fffffffull) return false;
        channel_stride = single_stride * frames;
        num_tiles = tiles_per_frame * frames;
        for (uint32_t f = 1; f < frames; ++f)                           // the other frames' tiles: the same offsets, one frame on
            for (uint32_t t = 0; t < tiles_per_frame; ++t) {
                tile_off_x.push_back(tile_off_x[t] + f * single_stride);
                tile_off_y.push_back(masked ? ((((tile_off_y[t] & 0xffffu) + f * (single_stride >> 2)) & 0xffffu) | (tile_off_y[t] & 0xffff0000u))
                                            : tile_off_y[t] + f * single_stride);
            }
        return true;
    }
    // element of pixel (y, x) of channel plane `ch`
    uint64_t offset(uint32_t ch, uint32_t y, uint32_t x) const { return (uint64_t)ch * channel_stride + (uint64_t)(y + 1u) * W_pad + 4u + x; }
    // gather offset of tap (dy, dx), dy, dx >= -1, relative to a tile's tile_off_x, for the plane starting at `plane`
    uint64_t tap(uint64_t plane, int dy, int dx) const { return plane + (uint64_t)(1 + dy) * W_pad + (uint64_t)(1 + dx); }
};

// ---- hardware presets (wavec/k44_plan_types.hpp:192-310); only name and unit count are surfaced ----
struct TargetPreset {
    std::string name = "b200";
    uint32_t num_units = 148;
};

inline TargetPreset preset_from_name(const char *p) {
    std::string s = p ? p : "auto";
    for (auto &c : s) c = (char)std::tolower((unsigned char)c);
    if (s == "rtx6000ada" || s == "rtx6000_ada" || s == "rtx6000" || s == "ada" || s == "sm_89" || s == "l40s")
        return {"rtx6000ada", 142};
    if (s == "rtx4090" || s == "4090") return {"rtx4090", 128};
    if (s == "h100" || s == "sm_90" || s == "hopper") return {"h100", 132};
    if (s == "rx9060xt") return {"rx9060xt", 32};
    // "auto", "b200", "blackwell", "sm_100", "sm_100a" and anything unknown: this library only targets B200
    return {"b200", 148};
}

// ---- 16x16-tile ("WMMA") weight order of the .tcff container -------------------------------------
// Bijection on 16-byte vectors (wavec/k44_plan_types.hpp:363-394): the vector of neuron j holding
// synapses [8*k8, 8*k8+8) is stored at  ((j/16)*(B/16) + k8/2)*32 + (k8&1)*16 + (j&15).
inline uint64_t wmma_vec_index(uint32_t j, uint32_t k8, uint32_t B) {
    return ((uint64_t)(j >> 4) * (B >> 4) + (k8 >> 1)) * 32u + ((k8 & 1u) << 4) + (j & 15u);
}

inline void rowmajor_to_wmma(const uint16_t *src, uint16_t *dst, uint32_t cout, uint32_t B) {
    const uint32_t v = B / 8u;
    for (uint32_t j = 0; j < cout; ++j)
        for (uint32_t k8 = 0; k8 < v; ++k8)
            std::memcpy(dst + wmma_vec_index(j, k8, B) * 8u, src + ((uint64_t)j * v + k8) * 8u, 16);
}

inline void wmma_to_rowmajor(const uint16_t *src, uint16_t *dst, uint32_t cout, uint32_t B) {
    const uint32_t v = B / 8u;
    for (uint32_t j = 0; j < cout; ++j)
        for (uint32_t k8 = 0; k8 < v; ++k8)
            std::memcpy(dst + ((uint64_t)j * v + k8) * 8u, src + wmma_vec_index(j, k8, B) * 8u, 16);
}

// ---- FNV-1a 64 (wavec/k44_tcff_io.hpp:10-17) -----------------------------------------------------
inline uint64_t fnv1a64(const uint8_t *p, size_t n) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < n; ++i) h = (h ^ p[i]) * 0x100000001b3ull;
    return h;
}

// ---- wave and plan --------------------------------------------------------------------------------
struct HostWave {
    std::string name;
    uint32_t cout = 0;             // padded rows
    uint32_t logical_cout = 0;
    uint32_t cin = 0;
    uint32_t group = 128;          // neurons per shared gather list ("cluster size" S)
    uint32_t fan_in = 0;           // B, padded
    uint32_t fan_in_raw = 0;
    int act = ACT_NONE;
    bool has_bias = true;
    bool has_residual = false;
    uint32_t weight_bits = 16;
    uint64_t y_off = 0, src_off = 0, res_off = 0, x_base_off = 0;
    uint32_t h_out = 1, w_out = 1;
    double gflops = 0.0;
    std::vector<uint16_t> w_wmma;      // [cout*fan_in] halves in container order (may be empty)
    std::vector<uint32_t> idx;         // [cout/group][fan_in] element offsets
    std::vector<uint16_t> bias;        // [cout]
    std::vector<uint16_t> cout_map;    // [cout] or empty
    // Large plans built in memory may keep their weights on the device (row-major [cout][fan_in])
    // and describe connectivity as runs of consecutive rows instead of an expanded table.
    const void *dev_weights_rowmajor = nullptr;
    uint32_t run_len = 0;              // rows per run when `run_rows` is used
    std::vector<uint32_t> run_rows;    // [cout/group][fan_in/run_len] first row of every run
    // Token shift: one entry per synapse (idx form) or per run (run form); empty = no shifts.
    std::vector<uint8_t> shifts;
    uint32_t frame_len = 0;            // columns per frame for the causal zero padding; 0 = whole row
    // Commands that are not waves (K44ExecCmd types RMSNORM / SWIGLU / ROPE_GQA_ATTN of the reference,
    // wavec/k44_plan_types.hpp:603-650): kind != 0, `cout` = channels of the main operand, `bias` = gamma (RMSNorm),
    // src_off / src2_off / src3_off = x | gate, up | q, k, v, y_off = destination.
    int kind = 0;                      // 0 wave, 1 RMSNorm, 2 SwiGLU product, 3 rotary + causal attention, 4 decode attention (cache),
                                       // 5 embedding gather (table in device memory), 6 arg-max over rows (greedy sampling)
    const void *dev_table = nullptr;   // kind 5: FP16 [vocab][cout] row-major, device memory, owned by the caller
    uint32_t vocab = 0;
    bool advance = false;              // kind 6: feed the result back as the next tokens and advance the decode position
    uint64_t src2_off = 0, src3_off = 0, kcache_off = 0, vcache_off = 0;
    float eps = 1e-5f, rope_theta = 10000.0f;
    uint32_t h_q = 0, h_kv = 0, head_dim = 0, seq_len = 0, max_seq = 0;
    bool llama3_scaling = false;
    // 2-D image waves and commands (kinds 7..12): the layout of the tensor the tiles walk over. pitch2d != 0 marks them:
    // rows are `pitch2d` (a plane's channel stride) apart instead of the plan's row pitch, and tile t reads from
    // tile_off_x[t] and writes to tile_off_y[t] (packed with a quad mask when `tile_mask`), see Layout2D.
    uint32_t pitch2d = 0;
    bool tile_mask = false;
    std::vector<uint32_t> tile_off_x, tile_off_y;
    //   kind 7 max-pool 2x2 stride 2, 8 max-pool 5x5 stride 1 pad 2, 9 nearest upsample x2, 10 space-to-depth 2x2,
    //   11 scatter of a 2x2 transposed convolution's four phase planes, 12 halo clear: `cout` planes from src_off
    //   (geometry `in2d`) to y_off (geometry `out2d`)
    struct Geom2D { uint32_t H = 0, W = 0, W_pad = 0, ch_stride = 0, frames = 1, frame_stride = 0; } in2d, out2d;
};

struct HostPlan {
    uint32_t batch_size = 1;
    Layout1D layout;                   // every tensor of a 1-D plan shares this layout
    uint64_t canvas_elems = 0;
    uint64_t total_w_bytes = 0, total_idx_bytes = 0;
    double total_gflops = 0.0, single_frame_gflops = 0.0;
    uint64_t input_off = 0;
    uint32_t input_c = 0, input_h = 1, input_w = 1;
    uint64_t output_off = 0;
    uint32_t output_c = 0, logical_output_c = 0, output_h = 1, output_w = 1;
    bool reuse_canvas = false;
    TargetPreset target;
    std::vector<HostWave> waves;
    // 2-D image plans: geometry of the input and output tensors (dense [C][H][W] at the boundary, haloed planes in the canvas)
    bool is_2d = false;
    HostWave::Geom2D in2d, out2d;
};

}  // namespace k44b
