/* Native additions of libk44wavec.so: build a wave plan from arrays or a .tcff file, keep inputs and
 * outputs on the device, run on a caller-supplied CUDA stream.
 *
 * These have no counterpart in the reference ABI; they exist because the reference's only execution
 * entry point (wavec_gpu_infer_f32, wavec/k44_wave_executor.cu:972-986) moves every input and output
 * through host FP32 arrays with blocking copies (:146-176), which would dominate the wave time.
 * Plan fields mirror K44ExecCmd / K44WavePlan (wavec/k44_plan_types.hpp:603-693).
 *
 * All functions return 0 on success and a negative value on failure unless stated otherwise; the
 * message of the last failure on the calling thread is returned by k44b_last_error().
 */
#ifndef K44B_H
#define K44B_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct k44b_wave_desc {
    uint32_t cout;            /* padded output rows, multiple of 16 (K44ExecCmd::Cout) */
    uint32_t logical_cout;    /* rows that carry neurons (K44ExecCmd::logical_Cout) */
    uint32_t cin;             /* informational (K44ExecCmd::Cin) */
    uint32_t group;           /* neurons sharing one gather list (K44ExecCmd::cluster_size) */
    uint32_t fan_in;          /* padded synapses per neuron, multiple of 8 (K44ExecCmd::B) */
    uint32_t fan_in_raw;      /* slots >= fan_in_raw must carry zero weights (K44ExecCmd::B_raw) */
    int32_t act;              /* 0 none, 1 relu, 2 sigmoid, 3 silu, 4 leaky-relu(0.1), 5 gelu (erf form; the tensor-core kernels use a fit within 2.6e-5 of it) */
    uint32_t has_residual;
    uint64_t y_off;           /* canvas element offset of output row 0 */
    uint64_t src_off;         /* informational */
    uint64_t res_off;         /* canvas element offset of residual row 0 */
    uint64_t x_base_off;      /* added to every entry of idx */
    const uint32_t *idx;      /* host [cout/group][fan_in] FP16-element offsets, or NULL when run_rows is given */
    const uint32_t *run_rows; /* host [cout/group][fan_in/run_len] first canvas row of every run, or NULL */
    uint32_t run_len;         /* rows per run (run_rows form) */
    uint32_t weights_on_device; /* 0: `weights` is a host pointer, 1: device pointer on the plan's device */
    const uint16_t *weights;  /* row-major [cout][fan_in] FP16 bit patterns */
    const uint16_t *bias;     /* host [cout] FP16 or NULL */
    const uint16_t *cout_map; /* host [cout] logical row -> stored row, or NULL */
    const char *name;         /* optional */
    /* Receptive-field token shift (optional): entry s of a group (one per synapse when `idx` is given, one per
     * run when `run_rows` is given) reads its row that many columns earlier; columns whose position inside
     * their frame of `frame_len` columns (0 = the whole row) is below the shift read zero. */
    const uint8_t *shifts;
    uint32_t frame_len;
    /* 2-D image planes (optional; K44ResDesc tile tables, wavec/k44_plan_types.hpp:517-569): with num_tiles != 0 the wave walks
     * `num_tiles` tiles of 64 consecutive elements of a plane; tile t gathers relative to tile_off_x[t] and stores at
     * tile_off_y[t] — or, with tile_mask != 0, at 4 * (tile_off_y[t] & 0xffff), writing only the 4-element quads whose bit
     * 16 + q of tile_off_y[t] is set; output (and residual) rows are `plane_stride` elements apart. `idx` is required (tap
     * offsets, any alignment); such waves run on the general kernels. */
    const uint32_t *tile_off_x;
    const uint32_t *tile_off_y;
    uint32_t num_tiles;
    uint32_t tile_mask;
    uint32_t plane_stride;
} k44b_wave_desc;

/* geometry of a haloed image plane set: pixel (y, x) of plane c at c * plane_stride + (y + 1) * w_pad + 4 + x */
typedef struct k44b_plane_geom { uint32_t h, w, w_pad, plane_stride; } k44b_plane_geom;

typedef struct k44b_wave_info_t {
    uint32_t cout, group, fan_in, box_rows;   /* box_rows: canvas rows per gather-table entry (8..64: tensor boxes; 1: single rows), 0 on the index path */
    int32_t path;                             /* 0 FP32-FMA kernel, 1 tcgen05 kernels, 2 element-wise / attention command, 3 general kernel on mma.sync */
    uint32_t n_tile;                          /* columns per tile on the tcgen05 path */
    uint32_t k_splits;                        /* K splits per tile (partial sums meet in FP32 scratch) */
    uint64_t synapses;                        /* logical_cout * fan_in_raw */
    uint64_t weight_bytes;                    /* packed size on the device */
    uint32_t m_blocks;                        /* 128-neuron blocks per tile on the streaming tcgen05 kernel (2: tiles of 256 neurons) */
    uint32_t cta_pairs;                       /* 1: those two blocks sit on a pair of CTAs (M = 256 MMAs) */
    uint32_t weights_in_tmem;                 /* token-shift kernel holding a work item's weight tile in tensor memory: column tiles per work item (0: not that kernel) */
    uint32_t reserved0;
} k44b_wave_info_t;

/* Create an empty plan bound to `device`: allocates and zeroes the canvas (canvas_elems FP16, rows of
 * `pitch` elements, pitch a multiple of 64). force_path: -1 automatic, 0 FMA kernel only, 1 tcgen05
 * wherever the gather structure allows. Returns NULL on failure. */
void *k44b_plan_create(int device, uint64_t canvas_elems, uint32_t pitch, uint32_t columns, int force_path);
/* Pack one wave onto the device (weights re-tiled, gather table analysed into row runs). Host and
 * device source arrays may be released when the call returns. */
int k44b_plan_add_wave(void *plan, const k44b_wave_desc *wave);
/* Declare the dense input / output tensors used by k44b_infer_f32. */
int k44b_plan_set_io(void *plan, uint64_t input_off, uint32_t input_c, uint64_t output_off, uint32_t output_c, uint32_t width);
/* Build a pure-wave plan from a TCFFv1.0 file (pitch from its geometry tag, else pitch_hint). */
void *k44b_plan_from_tcff(const char *path, uint32_t pitch_hint, int device, int force_path);
void k44b_plan_destroy(void *plan);

/* Device pointer to canvas element 0 (FP16). Valid until the plan is destroyed. */
void *k44b_canvas_ptr(void *plan);
uint64_t k44b_canvas_elems(void *plan);
int k44b_num_waves(void *plan);
int k44b_wave_info(void *plan, int wave, k44b_wave_info_t *out);
/* Queue every wave on `stream` (a cudaStream_t; NULL = default stream). Does not synchronise. */
int k44b_execute(void *plan, void *stream);
/* Same as k44b_execute, but the wave list is captured once into a CUDA graph and replayed with a single
 * launch. The first call on a plan builds the graph (do not issue it inside a stream capture). */
int k44b_execute_graph(void *plan, void *stream);
/* Queue one wave (0-based) on `stream`. */
int k44b_execute_wave(void *plan, int wave, void *stream);
/* Host FP16 in / out in canvas layout: h_in is [input_c][pitch], h_out is [output_c][pitch] (either may be
 * NULL to skip that copy). Copies and waves run on `stream`; returns once the output has arrived.
 * out_gpu_ms = device time of the waves only. Use pinned host memory for asynchronous copies. */
int k44b_infer_f16(void *plan, const uint16_t *h_in, uint16_t *h_out, float *out_gpu_ms, void *stream);
/* The same for a stream of inferences whose uploads should run under the previous inference's waves (the host link is the
 * bottleneck of plans with large inputs): k44b_infer_f16_begin starts the upload of an input into a staging buffer of
 * input_c * pitch * 2 bytes (allocated at the first call) on the plan's own copy stream and returns at once;
 * k44b_infer_f16_next completes the inference whose input is staged — device copy into the canvas, waves, output download on
 * `stream`, blocking like k44b_infer_f16 — and, if h_in_next is not NULL, starts the next upload before it waits. h_in must
 * stay valid until the k44b_infer_f16_next call that consumes it returns. -1 when nothing is staged / the staging is occupied.
 * No counterpart in the reference (wavec_gpu_infer_f32 is one blocking call, wavec/k44_wave_executor.cu:972-986). */
int k44b_infer_f16_begin(void *plan, const uint16_t *h_in);
int k44b_infer_f16_next(void *plan, const uint16_t *h_in_next, uint16_t *h_out, float *out_gpu_ms, void *stream);
/* Synchronise the plan's device and fetch-and-clear the kernels' status word (0 = ok). Returns -1 and
 * sets the error text when the status is non-zero. */
int k44b_status(void *plan, uint32_t *status);
/* Same contract as wavec_gpu_infer_f32 for a native plan. */
int k44b_infer_f32(void *plan, const float *h_in, int in_elems, float *h_out, int out_elems, float *out_gpu_ms);
/* ---- element-wise / attention commands between waves (the reference's RMSNORM, SWIGLU and ROPE_GQA_ATTN command
 * types, wavec/k44_plan_types.hpp:603-650, kernels/common/kernel44_valu_pack.cuh:104-248). Offsets are FP16 element
 * offsets of channel-major tensors in the canvas (multiples of 8); commands run in the order they were added, interleaved
 * with the waves. gamma_f16 may be null (no scale). Rotary embedding rotates q and k IN PLACE (half-split pairs), then
 * every column attends causally to the columns of its own sequence (blocks of seq_len columns, seq_len % 32 == 0).
 * head_dim 64 or 128. add_decode_attn has no counterpart in the reference (which reserves a key / value cache but never
 * reads it): one new token per column at the position set by k44b_plan_set_decode_pos — q and k are rotated at that
 * position, k and v are appended to the caches ([h_kv][max_seq][pitch][head_dim] regions of the canvas: the head_dim values of
 * one head, position and column are contiguous) and
 * the column attends to cache positions 0..pos. The position lives in device memory, so a captured graph can be replayed
 * for every position. */
int k44b_plan_add_rmsnorm(void *plan, const char *name, uint64_t src_off, uint64_t dst_off, uint32_t dim, float eps, const uint16_t *gamma_f16);
int k44b_plan_add_swiglu(void *plan, const char *name, uint64_t gate_off, uint64_t up_off, uint64_t dst_off, uint32_t rows);
int k44b_plan_add_rope_attn(void *plan, const char *name, uint64_t q_off, uint64_t k_off, uint64_t v_off, uint64_t out_off, uint32_t h_q,
                            uint32_t h_kv, uint32_t head_dim, float rope_theta, int llama3_scaling, uint32_t seq_len);
int k44b_plan_add_decode_attn(void *plan, const char *name, uint64_t q_off, uint64_t k_off, uint64_t v_off, uint64_t out_off,
                              uint64_t kcache_off, uint64_t vcache_off, uint32_t h_q, uint32_t h_kv, uint32_t head_dim, uint32_t max_seq,
                              float rope_theta, int llama3_scaling);
int k44b_plan_set_decode_pos(void *plan, int pos, void *stream);
/* Weight-free image commands between waves (kernels/common/kernel44_valu_pack.cuh:30-103), on `planes` channel planes from
 * src_off (geometry `in`) to dst_off (geometry `out`); offsets are canvas elements. op: 7 max-pool 2x2 stride 2, 8 max-pool 5x5
 * stride 1 pad 2, 9 nearest upsample x2, 10 space-to-depth 2x2 (`planes` input channels -> 4 * planes half-resolution planes
 * 4c + 2 * row parity + column parity), 11 scatter of the four phase planes q * planes + c of a 2x2 transposed convolution
 * into `planes` double-resolution planes, 12 halo clear of the destination planes (`in` ignored). */
int k44b_plan_add_image_op(void *plan, int op, const char *name, uint64_t src_off, uint64_t dst_off, uint32_t planes,
                           const k44b_plane_geom *in, const k44b_plane_geom *out);
/* Token I/O on the device (no counterpart in the reference, whose boundary is host F32 tensors): an embedding gather —
 * column b of the destination becomes row tokens[b] of an FP16 table [vocab][dim] that the caller keeps in device memory —
 * and a greedy arg-max over the rows of a tensor per column (lowest row wins ties). With advance != 0 the arg-max also
 * stores its result as the next step's tokens and moves the decode position on by one (saturating at max_seq - 1), so a
 * captured graph generates token after token without the host. set_tokens / get_next_tokens copy `n` 32-bit ids
 * (get_next_tokens synchronises the stream). */
int k44b_plan_add_embedding(void *plan, const char *name, const void *d_table_f16, uint32_t vocab, uint32_t dim, uint64_t dst_off);
int k44b_plan_add_argmax(void *plan, const char *name, uint64_t src_off, uint32_t rows, int advance, uint32_t max_seq);
int k44b_plan_set_tokens(void *plan, const int32_t *h_tokens, uint32_t n, void *stream);
int k44b_plan_get_next_tokens(void *plan, int32_t *h_tokens, uint32_t n, void *stream);

/* ---- neuron sharding over the GPUs of one box (no counterpart in the reference, which is single-GPU) ----
 * Every rank holds a plan with its rows of every wave and a full-size canvas. After k44b_plan_set_peers_* the wave
 * kernels store each output row into the rank's own canvas and into the peers' canvases (peer-mapped memory over
 * NVLink; the streaming tcgen05 kernel sends whole 128-row x 64-column tiles with tensor copies out of shared memory,
 * the other kernels 16-byte pieces), and a launch starts reading only when every peer has finished the launches before
 * it (one 32-bit word per peer, bounded wait: status bit 5 on expiry). All ranks must issue the same sequence of launches.
 * Rank r must hold rows [r * cout / world, (r + 1) * cout / world) of every wave. Supported for waves
 * that run on the tcgen05 kernels or on the mma.sync kernel (small neuron groups); plans with token-shifted waves,
 * element-wise commands or waves forced onto the FP32-FMA kernel are rejected. world <= 8.
 *   ipc_handles:    64-byte CUDA IPC handles of this plan's canvas and sync block, to be sent to the other processes
 *   set_peers_ipc:  `world` handles each (indexed by rank; the own entries are ignored), opened with peer access
 *   set_peers_raw:  the same with device pointers that are already valid on this GPU (same process)            */
int k44b_plan_ipc_handles(void *plan, void *canvas_handle64, void *sync_handle64);
int k44b_plan_set_peers_ipc(void *plan, int rank, int world, const void *canvas_handles, const void *sync_handles);
int k44b_plan_set_peers_raw(void *plan, int rank, int world, void *const *canvas_ptrs, void *const *sync_ptrs);
void *k44b_plan_sync_ptr(void *plan);
/* Launch ordering by region instead of by launch count (optional, after set_peers_*). A step of the plan is a fixed
 * sequence of launches (waves that cannot observe each other share one). launch_hulls writes, per launch, the canvas
 * element intervals it may read and write: out[launch][4] = {read_lo, read_hi, write_lo, write_hi}, half-open. The
 * caller collects the tables of all ranks and passes them, [world][launches][4], to set_peer_hulls on every rank; from
 * then on a launch waits only for the peers' nearest earlier launch that it depends on (whose rows it reads, whose reads
 * it overwrites, or whose rows it overwrites — on any rank, across step boundaries too) instead of for all of them.
 * Without this call every launch waits for all earlier launches of every peer. compute_peer_slack is the host arithmetic
 * behind it: out_slack[launch] = how many of the launches just before it need not be waited for. */
/* Signalling round trip between this rank and one peer (after set_peers_*; both ranks call it with the same iters and
 * payload_bytes, exactly one of them with initiator != 0, and no other work of the plan in flight): `iters` times a payload
 * (payload_bytes, a multiple of 16, stored at the start of the peer's canvas — use a scratch plan; 0 for none), one
 * system-scope fence and one count word, answered the same way by the peer. This is the sequence a sharded launch ends and
 * the next one starts with, so the result (nanoseconds per round trip; the call waits for `stream`) is the floor of what
 * each dependent launch of a sharded step costs. Bounded waits: fails with a message if the peer does not answer. */
int k44b_plan_peer_latency(void *plan, int peer_rank, int initiator, uint32_t iters, uint32_t payload_bytes, float *out_ns_per_round_trip, void *stream);
int k44b_plan_num_launches(void *plan);
int k44b_plan_launch_hulls(void *plan, uint64_t *out, uint64_t capacity_launches);
int k44b_plan_set_peer_hulls(void *plan, int world, const uint64_t *hulls, uint64_t launches);
void k44b_compute_peer_slack(const uint64_t *hulls, int world, uint64_t launches, uint32_t *out_slack);

/* Number of kernels this plan has launched so far. */
uint64_t k44b_launch_count(void *plan);
/* Unpack wave `wave`'s device weights to row-major [cout][fan_in] FP16 at device pointer d_dst. */
int k44b_wave_weights_rowmajor(void *plan, int wave, void *d_dst);

/* One tensor-core wave that allocates nothing. This entry point has no counterpart in the reference.
 *
 * For callers that may not let the library allocate device memory: processes whose HBM is entirely owned by
 * the host framework's arena, callers under a fixed memory budget, and latency-critical sections that cannot
 * take the device-wide synchronisation of cudaMalloc / cudaFree. Everything the wave touches is passed in as
 * device pointers owned by the caller; the split-K partial sums, arrival counters and status word live in a
 * fixed array inside the library image (about 2 MiB per GPU, present for the life of the process).
 *
 *   d_canvas         FP16 canvas holding the gathered rows and receiving the output rows (rows of `pitch`)
 *   d_weights_tiled  weights in the library's packed order: [cout/128 rounded up][ceil(fan_in/64)] blocks of
 *                    16 KiB; inside a block neuron row r (0..127) is 128 bytes and the 16-byte chunk c of its 64
 *                    synapses sits at chunk position c ^ (r & 7); rows >= cout and synapses >= fan_in are zero
 *   d_box_rows       [cout/group][ceil(fan_in/64) * 64/rows_per_box] first canvas row of every box of
 *                    `rows_per_box` consecutive rows (what k44b_analyze_gather returns)
 *   d_bias           [cout] FP16 or NULL;  act as in k44b_wave_desc;  y_off = element offset of output row 0
 *   k_splits         1..ceil(fan_in/64): how many CTAs share one output tile's fan-in
 *
 * Limits: (cout/128 rounded up) * (pitch/64) <= K44B_STATIC_MAX_TILES, otherwise the call fails with a message
 * naming the limit; no residual and no row map; the rows the wave gathers must not overlap the rows it writes.
 * The first call on a device resolves the array's address and sets kernel attributes. Every call queues its work
 * on `stream`, then waits for the stream and reads the kernel's status word back, so no call may be made while
 * `stream` is being captured (such a call is refused with a message). Every call uses the same array and clears
 * the part it needs first, so two calls that overlap on one GPU (different streams or threads) race.
 * Returns 0, or -1 with a message copied to `err` (if given). Calls no cudaMalloc / cudaFree. */
#define K44B_STATIC_MAX_TILES 64
int k44b_wave_forward_static(void *d_canvas, uint64_t canvas_elems, uint32_t pitch, const void *d_weights_tiled,
                             const uint32_t *d_box_rows, uint32_t rows_per_box, const uint16_t *d_bias, uint32_t cout, uint32_t group,
                             uint32_t fan_in, int act, uint64_t y_off, uint32_t k_splits, void *stream, char *err, uint32_t err_capacity);

/* Handle-based plans (wavec_*): device used by wavec_gpu_init_plan, and access to the executor's plan. */
int k44b_set_device(void *wavec_handle, int device);
int k44b_set_force_path(void *wavec_handle, int force_path);
void *k44b_handle_plan(void *wavec_handle);   /* plan pointer usable with the k44b_* calls above, or NULL */

/* Utilities */
const char *k44b_last_error(void);
const char *k44b_version(void);
/* dst[i] = FP16(scale * N(0,1)) from a stateless hash of (seed, i); dst is a device pointer. */
int k44b_fill_normal_f16(void *d_dst, uint64_t n, uint64_t seed, float scale, void *stream);
/* Host helpers (no device needed): FNV-1a-64, FP32->FP16 RTE, 16x16-tile weight order. */
uint64_t k44b_fnv1a64(const uint8_t *data, uint64_t len);
void k44b_f32_to_f16(const float *src, uint16_t *dst, uint64_t n);
void k44b_rowmajor_to_wmma(const uint16_t *src, uint16_t *dst, uint32_t cout, uint32_t fan_in);
void k44b_wmma_to_rowmajor(const uint16_t *src, uint16_t *dst, uint32_t cout, uint32_t fan_in);
/* Host-only gather analysis: returns the rows per table entry — 8/16/32/64 when the gather lists are runs of whole boxes
 * (fetched as tensor boxes), 1 when they are scattered single rows (one entry per synapse, fetched row by row) — or 0 when
 * the offsets are not whole rows (element-granular shifts: general kernels, index table); out_box_rows (optional, capacity
 * in entries) receives the table, padded per group to whole 64-synapse stages. */
int k44b_analyze_gather(const k44b_wave_desc *wave, uint32_t pitch, uint64_t canvas_elems, uint32_t *out_box_rows,
                        uint64_t capacity, uint64_t *out_count);

#ifdef __cplusplus
}
#endif
#endif
