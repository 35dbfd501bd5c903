// Device-side contracts of the wave kernels: packed weight layout, gather tables, launch wrappers.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

namespace k44b {

// ---- packed ("tiled") weight layout --------------------------------------------------------------
// Weights of a wave are stored as [m_tile][k_stage] blocks of 16 KiB: 128 neurons x 64 synapses of
// FP16, i.e. 128 rows of 128 bytes. Inside a block the 16-byte chunk c (0..7) of row r sits at chunk
// position c ^ (r & 7) — the 128-byte shared-memory swizzle — so that one linear bulk copy of a block
// lands in shared memory already in the K-major SWIZZLE_128B operand layout of tcgen05.mma.
// Rows >= cout and synapses >= fan_in are zero.
constexpr uint32_t kTileM = 128;       // neurons per tile
constexpr uint32_t kStageK = 64;       // synapses per pipeline stage
constexpr uint32_t kStageWBytes = kTileM * kStageK * 2;

__host__ __device__ inline uint64_t tiled_vec_index(uint32_t j, uint32_t k8, uint32_t num_kstages) {
    const uint32_t mt = j >> 7, r = j & 127u, ks = k8 >> 3, c = k8 & 7u;
    return (((uint64_t)mt * num_kstages + ks) * 128u + r) * 8u + (c ^ (r & 7u));
}

enum GatherMode : int {
    GATHER_IDX = 0,    // one 32-bit FP16-element offset per synapse (general; any alignment)
    GATHER_BOX = 1,    // runs of `box_h` consecutive rows: one 32-bit entry per box = row | token shift << 28
};
constexpr uint32_t kBoxRowMask = 0x0fffffffu;   // canvas row of a box entry; the top 4 bits carry its token shift (0..8)

enum WavePath : int { PATH_FMA = 0, PATH_UMMA = 1, PATH_AUX = 2, PATH_MMA = 3 };   // FP32 FMA | tcgen05 | element-wise command | mma.sync

// Status word written by kernels instead of trapping or hanging.
enum KernelStatus : uint32_t {
    ST_OK = 0,
    ST_TIMEOUT_PRODUCER = 1u << 0,
    ST_TIMEOUT_MMA = 1u << 1,
    ST_TIMEOUT_EPILOGUE = 1u << 2,
    ST_TIMEOUT_DRAIN = 1u << 3,
    ST_BAD_INDEX = 1u << 4,
    ST_TIMEOUT_PEER = 1u << 5,
};

// Neuron sharding over several GPUs: every rank stores the rows it computes into its own canvas and, at the same
// element offset, into the canvases of its peers (peer-mapped pointers over NVLink), so that each GPU's next wave
// gathers from a complete canvas in its own HBM. Launch n of a rank may start once every peer has finished its
// launches 0..n-1: the CTA that finishes a launch last publishes the rank's launch count into one word per peer
// (`arrive`), and the first thing a launch does with the canvas is a bounded wait for those words.
constexpr int kMaxPeers = 7;
struct PeerArgs {
    __half *canvas[kMaxPeers] = {};       // the peers' canvases
    uint32_t *arrive[kMaxPeers] = {};     // this rank's word in each peer's sync block
    uint32_t *sync = nullptr;             // own sync block: [0..6] the peers' launch counts, [8] CTAs done in the running launch, [9] launches completed
    uint32_t n_peers = 0;
};
constexpr uint32_t kSyncWords = 16, kSyncDone = 8, kSyncEpoch = 9, kSyncProbe = 10;   // [10] the latency probe's counter word, [12..13] its result

struct WaveArgs {
    // tensors
    const uint4 *w_tiles = nullptr;
    const uint32_t *gather = nullptr;     // idx table or box-row table
    const __half *bias = nullptr;         // may be null
    const uint16_t *cout_map = nullptr;   // may be null
    __half *canvas = nullptr;
    uint32_t *status = nullptr;
    // geometry
    uint64_t canvas_elems = 0;
    uint64_t y_off = 0, res_off = 0, x_base_off = 0;
    uint32_t cout = 0, group = 0, fan_in = 0;
    uint32_t mtiles_per_group = 1;        // 128-neuron tiles sharing one gather list (tensor-core path)
    uint32_t num_kstages = 0;             // ceil(fan_in / 64)
    uint32_t pitch = 0, num_col_tiles64 = 0;
    int gather_mode = GATHER_IDX;
    uint32_t box_h = 0, boxes_per_group = 0;
    int act = 0;
    int has_residual = 0;
    // receptive-field token shift: a synapse reads its row `shift` columns earlier; columns whose position inside
    // their frame is below the shift read zero
    const uint8_t *shifts = nullptr;      // per synapse (GATHER_IDX only; box entries carry their own shift)
    uint32_t frame_len = 0;               // columns per frame (0: the whole row)
    uint32_t has_shift = 0;
    // split-K (tensor-core path): partial sums meet in an FP32 scratch tile, the last arrival finishes the rows
    uint32_t k_splits = 1, kstages_per_split = 0;
    float *scratch = nullptr;             // [tiles][N_TILE][128] FP32, all zero between launches
    uint32_t *counters = nullptr;         // [tiles], all zero between launches
    // 2-D image waves (general kernels only): tile t gathers relative to tile_off_x[t] and stores at tile_off_y[t] inside a
    // plane instead of at 64 * t; with tile_mask the entry is (plane offset / 4) & 0xffff | mask << 16 and only the 4-element
    // quads whose mask bit is set are stored (wavec/k44_plan_types.hpp:517-569; kernels/cuda/kernel44_cuda_pack.cuh:116-123).
    // `pitch` is then the plane stride of the output tensor and num_col_tiles64 the number of tiles of a plane.
    const uint32_t *tile_off_x = nullptr, *tile_off_y = nullptr;
    uint32_t tile_mask = 0;
    const PeerArgs *peers = nullptr;      // device memory; null unless the plan is neuron-sharded over several GPUs
    uint32_t peer_slack = 0;              // sharded plans: how many of the peers' latest launches this launch need not wait for
    // Output through tensor copies (streaming tcgen05 kernel, waves without an output-row map): device array of tensor maps
    // over the wave's output rows, [cout][pitch] FP16 from y_off, boxes of 64 columns x 128 rows, 128-byte swizzle;
    // [0] = this rank's canvas, [1 .. n_out_maps-1] = the same rows in the peers' canvases. Null: stores from registers.
    const CUtensorMap *out_maps = nullptr;
    uint32_t n_out_maps = 0;
};

// Element-wise / attention steps between waves (k44_valu.cu)
enum AuxKind : int { AUX_NONE = 0, AUX_RMSNORM = 1, AUX_SWIGLU = 2, AUX_ROPE_ATTN = 3, AUX_DECODE_ATTN = 4, AUX_EMBED = 5, AUX_ARGMAX = 6,
                     // 2-D image glue on haloed planes (kernels/common/kernel44_valu_pack.cuh:30-103)
                     AUX_MAXPOOL2 = 7, AUX_MAXPOOL5 = 8, AUX_UPSAMPLE2 = 9, AUX_S2D = 10, AUX_UPCONV_SCATTER = 11, AUX_HALO_CLEAR = 12 };
struct AuxArgs {
    int kind = AUX_NONE;
    __half *canvas = nullptr;
    uint64_t src_off = 0, src2_off = 0, src3_off = 0, dst_off = 0;    // x | gate, up | q, k, v
    uint64_t kcache_off = 0, vcache_off = 0;                         // decode attention: [h_kv][max_seq][pitch][head_dim]
    uint32_t rows = 0, pitch = 0, columns = 0;
    float eps = 1e-5f;
    const __half *gamma = nullptr;                                   // device, [rows] or null
    uint32_t h_q = 0, h_kv = 0, head_dim = 0, seq_len = 0, max_seq = 0, llama3 = 0;
    float neg_log_theta = -9.210340371976184f;
    const int *pos_ptr = nullptr;                                    // decode: current position, device memory
    float *partial = nullptr;                                        // decode: per-chunk partial results [chunks][h_q][pitch][kDecodeRow]
    // token I/O: embedding gather (table FP16 [vocab][rows] row-major in device memory, one token id per column) and
    // greedy arg-max over the rows of a tensor (lowest row wins ties); `advance` also feeds the result back as the next
    // step's tokens and moves the decode position on by one (saturating at max_seq - 1)
    const __half *table = nullptr;
    uint32_t vocab = 0, advance = 0;
    int *tokens = nullptr, *next_tokens = nullptr, *pos_rw = nullptr;
    unsigned long long *argmax_scratch = nullptr;                    // [row chunks][pitch] packed (value key, row)
    // 2-D image commands: `rows` planes; source / destination geometry (pixels, padded row length, plane stride)
    uint32_t h_in = 0, w_in = 0, wpad_in = 0, cs_in = 0, h_out = 0, w_out = 0, wpad_out = 0, cs_out = 0;
    uint32_t frames = 1, fs_in = 0, fs_out = 0;      // frames per channel and their strides (cs = frames * fs)
};
constexpr uint32_t kArgmaxChunk = 256;                               // rows per arg-max CTA
constexpr uint32_t kDecodeChunk = 32;
constexpr uint32_t kDecodeRow = 68;                                  // floats per partial result: 64 values, maximum, sum, 2 pad (16-byte aligned rows)                                // cache positions per partial-attention CTA
cudaError_t launch_aux(const AuxArgs &a, bool dependent_launch, cudaStream_t s);
cudaError_t launch_image_aux(const AuxArgs &a, cudaStream_t s);       // kinds AUX_MAXPOOL2 .. AUX_HALO_CLEAR (k44_image.cu)

// Up to four mutually independent small waves launched as one grid (their clusters are numbered consecutively).
constexpr int kMaxGroupWaves = 4;
struct WaveGroupArgs {
    WaveArgs w[kMaxGroupWaves];
    uint32_t first_cluster[kMaxGroupWaves] = {0, 0, 0, 0};   // first cluster index of each wave
    uint32_t count = 0;                                       // waves in the group
    uint32_t splits = 1;                                      // K splits = cluster size, common to the group
    uint32_t total_clusters = 0;
};

// tcgen05 operand descriptors are assembled on the host (see k44_exec.cu) and passed in.
struct UmmaDesc {
    uint64_t a_base = 0, b_base = 0;      // descriptor bits without the start address
    uint32_t a_k_step = 0, b_k_step = 0;  // start-address increment per K=16 step, 16-byte units
    uint32_t idesc = 0;
    uint32_t n_tile = 64;
    uint32_t small_wave = 0;              // 1: 4-stage, two-CTAs-per-SM variant (N_TILE 64 only)
    unsigned long long wait_cycles = 0;   // bound for every barrier wait
    uint32_t rows_mode = 1;               // scattered single rows: 1 asynchronous 16-byte copies from four extra warps, 2 gather-mode tensor copies (measured slower)
    uint32_t pair = 0;                    // 1: the wave runs on CTA pairs (tiles of 256 neurons x 256 columns, M = 256 MMAs)
    uint32_t m_blocks = 1;                // 128-neuron blocks per tile: 2 = tiles of 256 neurons sharing one gathered operand (256-column tiles only)
    uint32_t ws_chunk = 0;                // token-shift kernel with the weights in tensor memory: column tiles per work item (0: not that kernel)
    uint32_t ws_groups = 2;               // ... and its groups of four aligner warps (1 or 2), each taking every ws_groups-th stage
};

cudaError_t launch_wave_fma(const WaveArgs &a, cudaStream_t s);
cudaError_t launch_wave_mma(const WaveArgs &a, unsigned long long wait_cycles, cudaStream_t s);   // general path on mma.sync (k44_mma_kernel.cu); wait_cycles bounds the peer wait
cudaError_t launch_wave_umma(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s);
// per tile width (k44_stream_n64.cu, _n128.cu, _n256.cu): launch, and opt-in to large dynamic shared memory
cudaError_t launch_wave_umma_n64(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s);
cudaError_t launch_wave_umma_n128(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s);
cudaError_t launch_wave_umma_n256(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s);
// tiles of 256 neurons x 256 columns on CTA pairs (k44_pair_kernel.cu); wmap: the packed weights as rows of 128 bytes, boxes of 128 rows
cudaError_t launch_wave_umma_pair(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, const CUtensorMap &wmap, int num_sms, cudaStream_t s);
cudaError_t umma_setup_n64();
cudaError_t umma_setup_n128();
cudaError_t umma_setup_n256();
// small waves: one item per CTA, the K splits of a tile form a cluster (k_splits in {1,2,4,8}) and reduce through
// distributed shared memory; dependent_launch adds the programmatic-dependent-launch attribute
cudaError_t launch_wave_umma_cluster(const WaveGroupArgs &g, const UmmaDesc &d, const CUtensorMap &tmap, bool dependent_launch, int num_sms, cudaStream_t s);
// token-shifted runs (box gather, shifts in the table entries): n_tile 64 or 128, frames must be whole tiles; the tensor
// map describes the canvas with boxes of (n_tile + 8) columns x box_h rows and no swizzle
cudaError_t launch_wave_umma_shift(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s);
// the same with the weight tile of a work item held in tensor memory (k44_shift_ws_kernel.cu): fan-in up to 512, tiles of 128 columns
cudaError_t launch_wave_umma_shift_ws(const WaveArgs &a, const UmmaDesc &d, const CUtensorMap &tmap, int num_sms, cudaStream_t s);
bool shift_ws_supported(const WaveArgs &a);
uint32_t shift_ws_chunk(uint32_t mtiles, uint32_t tiles_n, uint32_t num_sms);
cudaError_t mma_kernel_setup();        // same for the mma.sync kernel
cudaError_t umma_kernel_setup();       // opt in to large dynamic shared memory (once per device)

// signalling round trip between two sharded ranks (k44_peer.cu); d_out: [0] nanoseconds, [1] completed round trips
cudaError_t launch_peer_pingpong(uint32_t *own_word, uint32_t *peer_word, void *peer_payload, uint32_t payload_bytes, bool initiator, uint32_t iters,
                                 uint32_t base, unsigned long long wait_cycles, unsigned long long *d_out, cudaStream_t s);

// packer kernels
cudaError_t launch_repack_wmma_to_tiled(const uint4 *src_wmma, uint4 *dst, uint32_t cout, uint32_t fan_in, cudaStream_t s);
cudaError_t launch_repack_rowmajor_to_tiled(const uint4 *src_rows, uint4 *dst, uint32_t cout, uint32_t fan_in, cudaStream_t s);
cudaError_t launch_tiled_to_rowmajor(const uint4 *src_tiled, uint4 *dst_rows, uint32_t cout, uint32_t fan_in, cudaStream_t s);
// host f32 [C][W] <-> canvas rows (FP16, pitch), on the device
cudaError_t launch_f32_to_canvas(const float *src, __half *dst, uint32_t rows, uint32_t width, uint32_t pitch, cudaStream_t s);
cudaError_t launch_canvas_to_f32(const __half *src, float *dst, uint32_t rows, uint32_t width, uint32_t pitch, cudaStream_t s);
// dense F32 [C][H][W] <-> haloed FP16 planes (row length wpad, plane stride cs; pixel (y, x) at (y + 1) * wpad + 4 + x)
cudaError_t launch_f32_to_planes(const float *src, __half *dst, uint32_t c, uint32_t h, uint32_t w, uint32_t wpad, uint32_t cs, uint32_t frames, uint32_t fs, cudaStream_t s);
cudaError_t launch_planes_to_f32(const __half *src, float *dst, uint32_t c, uint32_t h, uint32_t w, uint32_t wpad, uint32_t cs, uint32_t frames, uint32_t fs, cudaStream_t s);
// counter-based normal fill: element i gets scale * N(0,1) from a stateless hash of (seed, i)
cudaError_t launch_fill_normal_f16(__half *dst, uint64_t n, uint64_t seed, float scale, cudaStream_t s);

}  // namespace k44b
