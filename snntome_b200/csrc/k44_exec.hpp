// Wave executor: owns the device copy of a plan (packed weights, gather tables, canvas) and runs the
// wave list. Counterpart of the reference's K44GpuExecutorState (wavec/k44_wave_executor.cu:265-619)
// with three differences that matter to callers: no call ever terminates the process (errors are
// returned with a message), execution can be queued on a caller-supplied stream, and the canvas can
// be reached as a device pointer so that inputs and outputs need not travel through host FP32.
#pragma once
#include <string>
#include <vector>

#include "k44_host.hpp"
#include "k44_kernels.cuh"

namespace k44b {

// Gather description derived from a wave's index table (or given directly as runs).
struct GatherPlan {
    bool box_ok = false;                 // every run is made of whole boxes of `box_h` rows
    bool small_group = false;            // groups of 16 / 32 / 64 neurons: boxes are usable, but only by the general kernels
    bool shared_by_all = false;          // all groups had the same list: the table holds it once
    uint32_t box_h = 0;                  // 8, 16, 32 or 64
    uint32_t boxes_per_group = 0;        // == 64/box_h * ceil(fan_in/64)
    std::vector<uint32_t> box_rows;      // [groups][boxes_per_group] canvas row | token shift << 28
    uint32_t max_shift = 0;              // largest token shift of any run
    std::string why_not;                 // reason the tensor-core path cannot be used
};

// Launch ordering of neuron-sharded plans. `hulls` holds, for every rank and every launch of a step, the canvas element
// intervals the launch may read and write: [world][launches][4] = {read_lo, read_hi, write_lo, write_hi} (half-open).
// A launch must wait until every peer has completed the nearest earlier launch (of the same step or, cyclically, of the
// step before) whose rows it reads, whose reads it overwrites or whose rows it overwrites, on any rank; the launches after
// that one may still be running on the peers. out_slack[n] = how many of the launches just before launch n need not be
// waited for (0 = wait for all of them). Pure host arithmetic.
void compute_peer_slack(const uint64_t *hulls, int world, size_t launches, uint32_t *out_slack);

// Pure host analysis (unit-testable without a device).
GatherPlan analyze_gather(const HostWave &w, uint32_t pitch, uint64_t canvas_elems);
bool validate_wave(const HostWave &w, uint32_t pitch, uint32_t num_tiles, uint64_t canvas_elems, std::string &err);
UmmaDesc make_umma_desc(uint32_t n_tile);

struct DeviceWave {
    std::string name;
    bool is_aux = false;                 // element-wise / attention step (k44_valu.cu) instead of a wave
    AuxArgs aux;
    WaveArgs args;
    UmmaDesc desc;
    CUtensorMap tmap;
    CUtensorMap wmap;                    // CTA-pair kernel: the packed weights as rows of 128 bytes
    int path = PATH_FMA;
    bool use_cluster = false;            // small wave: K splits form a cluster and reduce through shared memory
    bool use_shift = false;              // token-shifted runs: tensor-core kernel with aligner warps
    bool umma_capable = false;
    std::string fma_reason;
    void *d_weights = nullptr, *d_gather = nullptr, *d_bias = nullptr, *d_map = nullptr, *d_shifts = nullptr;
    void *d_out_maps = nullptr;          // output tensor maps (own canvas + peers) of a streaming tcgen05 wave
    uint32_t *d_idx_table = nullptr;     // expanded table kept for the FMA path when boxes are used too
    uint64_t synapses = 0;               // logical_cout * fan_in_raw
    uint64_t read_lo = 0, read_hi = 0;   // canvas element interval this wave may read (gathers and residual)
    uint64_t write_lo = 0, write_hi = 0; // canvas element interval it writes
    bool groupable = false;              // may share a launch with independent neighbours
    uint64_t weight_bytes = 0;
};

class Executor {
  public:
    static constexpr size_t kStatusBytes = 256;    // status word (padded)
    ~Executor() { release(); }
    std::string err;

    // force_path: -1 choose per wave, 0 always FMA, 1 tensor cores wherever the gather allows
    bool begin(int device, uint64_t canvas_elems, uint32_t pitch, uint32_t columns, int force_path);
    bool add_wave(const HostWave &w);
    bool add_aux(const HostWave &w);                               // HostWave::kind != 0
    bool add_wave_2d(const HostWave &w);                           // HostWave::pitch2d != 0: a wave over image planes
    int *tokens_ptr();                                             // device int32 [pitch]: token id per column (embedding gather input)
    int *next_tokens_ptr();                                        // device int32 [pitch]: result of the last arg-max command
    int *decode_pos_ptr();                                         // device word holding the position decode attention works at
    void set_io(uint64_t in_off, uint32_t in_c, uint64_t out_off, uint32_t out_c, uint32_t width);
    bool init(const HostPlan &plan, int device, int force_path);   // begin + add_wave* + set_io
    void release();

    bool execute(cudaStream_t stream);                             // queue every wave; no sync
    bool execute_wave(size_t wave, cudaStream_t stream);          // queue one wave; no sync
    bool execute_graph(cudaStream_t stream);                      // replay the wave list as one CUDA graph
    // host FP16 rows in canvas layout ([input_c][pitch] in, [output_c][pitch] out), copies on `stream`
    bool infer_f16(const uint16_t *h_in, uint16_t *h_out, float *gpu_ms, cudaStream_t stream);
    // the same with the next inference's upload running under this inference's waves (staging buffer + copy stream)
    bool infer_f16_begin(const uint16_t *h_in);
    bool infer_f16_next(const uint16_t *h_in_next, uint16_t *h_out, float *gpu_ms, cudaStream_t stream);
    bool execute_timed(float *ms);                                 // default stream, event-timed, synchronous
    bool infer_f32(const float *h_in, int in_elems, float *h_out, int out_elems, float *gpu_ms);
    bool read_status(uint32_t *status);                            // synchronises the device
    // Neuron sharding: exchange of wave rows by direct stores into the peers' canvases.
    bool ipc_handles(void *canvas_handle64, void *sync_handle64);    // handles of this plan's canvas and sync block for the other processes
    bool set_peers_ipc(int rank, int world, const void *canvas_handles, const void *sync_handles);   // world x 64 bytes each, indexed by rank
    bool set_peers_raw(int rank, int world, void *const *canvas_ptrs, void *const *sync_ptrs);       // device pointers valid on this GPU, indexed by rank
    void *sync_ptr();
    // Signalling round trip with one peer (both ranks call this with the same iters / payload, one of them as initiator):
    // `iters` times a payload of payload_bytes (a multiple of 16, written to the start of the peer's canvas; 0 = none), a
    // system-scope fence and a count word, answered the same way. Synchronises `stream`; returns nanoseconds per round trip.
    bool peer_latency(int peer_rank, bool initiator, uint32_t iters, uint32_t payload_bytes, float *ns_per_round_trip, cudaStream_t stream);
    // launches per step (waves that share a launch count once) and their read / write intervals, [launches][4] as above
    size_t num_launches();
    bool launch_hulls(uint64_t *out, size_t capacity);
    // the same table from every rank, [world][launches][4]: lets launches skip the wait for peers' launches they do not depend on
    bool set_peer_hulls(int world, const uint64_t *hulls, size_t launches);
    bool weights_to_rowmajor(size_t wave, void *d_dst);            // unpack check: tiled -> [cout][fan_in]

    bool ready() const { return canvas_ != nullptr; }
    __half *canvas() const { return canvas_; }
    uint64_t canvas_elems() const { return canvas_elems_; }
    size_t num_waves() const { return waves_.size(); }
    const DeviceWave &wave(size_t i) const { return waves_[i]; }
    int device() const { return device_; }
    uint32_t pitch() const { return pitch_; }
    uint64_t launches() const { return launches_; }

  private:
    bool fail(const std::string &m) { err = m; return false; }
    bool check(cudaError_t e, const char *what);
    bool make_tensor_map(DeviceWave &dw, uint32_t box_cols, bool swizzle128);
    bool encode_map(CUtensorMap *map, void *base, uint64_t rows, uint32_t box_cols, uint32_t box_rows, bool swizzle128);
    bool upload_out_maps(DeviceWave &dw, void *const *peer_canvases, uint32_t n);
    bool reserve_scratch(size_t tiles);
    void recover_after_abort();
    bool launch_one(DeviceWave &w, cudaStream_t stream, uint32_t peer_slack = 0);
    void drop_graph();
    void build_groups();
    bool launch_group(size_t gi, cudaStream_t stream);
    struct LaunchGroup { std::vector<size_t> waves; WaveGroupArgs args; uint32_t peer_slack = 0; };
    std::vector<uint32_t> peer_slack_;   // per launch of a step; empty: every launch waits for all earlier ones
    std::vector<LaunchGroup> groups_;
    bool groups_valid_ = false;

    int device_ = -1, num_sms_ = 148, force_path_ = -1;
    __half *canvas_ = nullptr;
    uint64_t canvas_elems_ = 0;
    uint32_t pitch_ = 0, columns_ = 0;
    uint32_t *d_status_ = nullptr;
    std::vector<DeviceWave> waves_;
    uint64_t in_off_ = 0, out_off_ = 0;
    uint32_t in_c_ = 0, out_c_ = 0, io_width_ = 0;
    float *d_in_f32_ = nullptr, *d_out_f32_ = nullptr;
    cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
    __half *d_stage_in_ = nullptr;                  // staging copy of the input rows for pipelined host I/O
    cudaStream_t copy_stream_ = nullptr;
    cudaEvent_t ev_uploaded_ = nullptr, ev_stage_free_ = nullptr;
    bool stage_pending_ = false;
    uint64_t launches_ = 0;
    float *d_scratch_ = nullptr;
    uint32_t *d_counters_ = nullptr;
    int *d_pos_ = nullptr;                // decode position
    int *d_tokens_ = nullptr, *d_next_tokens_ = nullptr;
    unsigned long long *d_argmax_ = nullptr;
    size_t argmax_words_ = 0;
    float *d_decode_partial_ = nullptr;   // per-chunk partial attention results, shared by all decode-attention commands
    size_t decode_partial_bytes_ = 0;
    // neuron sharding over several GPUs (see PeerArgs)
    uint32_t *d_sync_ = nullptr;          // kSyncWords words, allocated on first use
    PeerArgs *d_peers_ = nullptr;
    std::vector<void *> ipc_opened_;      // peer mappings to close on release
    int peer_rank_ = 0, peer_world_ = 1;
    bool is_2d_ = false;                 // image plan: dense [C][H][W] at the host boundary, haloed planes in the canvas
    HostWave::Geom2D in2d_, out2d_;
    std::vector<void *> peer_canvas_, peer_sync_;   // indexed by rank (own entries null)
    uint32_t probe_base_ = 0;
    size_t scratch_tiles_ = 0;
    cudaGraphExec_t graph_exec_ = nullptr;
    bool pdl_ = true;                    // programmatic dependent launch between consecutive small waves
};

const char *status_string(uint32_t st);

}  // namespace k44b
