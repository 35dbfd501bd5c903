// Plan -> device packer and wave scheduler (see k44_exec.hpp).
#include "k44_exec.hpp"

#include <cstdlib>

namespace k44b {

const char *status_string(uint32_t st) {
    if (st == 0) return "ok";
    if (st & ST_BAD_INDEX) return "gather offset outside the canvas";
    if (st & ST_TIMEOUT_PEER) return "timed out waiting for a peer GPU's rows";
    if (st & ST_TIMEOUT_DRAIN) return "timed out draining in-flight copies";
    if (st & ST_TIMEOUT_PRODUCER) return "producer timed out waiting for a free stage";
    if (st & ST_TIMEOUT_MMA) return "MMA issuer timed out waiting for operands";
    if (st & ST_TIMEOUT_EPILOGUE) return "epilogue timed out waiting for an accumulator";
    return "unknown kernel status";
}

// ---------------------------------------------------------------------------------------------------
// host analysis
// ---------------------------------------------------------------------------------------------------
bool validate_wave(const HostWave &w, uint32_t pitch, uint32_t num_tiles, uint64_t canvas_elems, std::string &err) {
    auto bad = [&](const std::string &m) { err = "wave '" + w.name + "': " + m; return false; };
    if (w.cout == 0 || w.cout % 16u) return bad("row count must be a positive multiple of 16");
    if (w.group == 0 || w.cout % w.group) return bad("group size must divide the row count");
    if (w.fan_in == 0 || w.fan_in % 8u) return bad("fan-in must be a positive multiple of 8");
    if (w.fan_in_raw > w.fan_in) return bad("raw fan-in exceeds the padded fan-in");
    if (pitch == 0 || pitch % 64u || num_tiles * 64u != pitch) return bad("row pitch must be a multiple of 64");
    if (w.y_off % 8u || w.res_off % 8u) return bad("output / residual offsets must be multiples of 8 elements");
    if (w.y_off + (uint64_t)w.cout * pitch > canvas_elems) return bad("output rows leave the canvas");
    if (w.has_residual && w.res_off + (uint64_t)w.cout * pitch > canvas_elems) return bad("residual rows leave the canvas");
    const uint32_t groups = w.cout / w.group;
    if (!w.run_rows.empty()) {
        if (w.run_len == 0 || w.fan_in % w.run_len) return bad("run length must divide the fan-in");
        if (w.run_rows.size() != (size_t)groups * (w.fan_in / w.run_len)) return bad("run table has the wrong size");
        const uint64_t rows = canvas_elems / pitch;
        for (uint32_t r : w.run_rows)
            if ((uint64_t)r + w.run_len > rows) return bad("a run leaves the canvas");
    } else {
        if (w.idx.size() != (size_t)groups * w.fan_in) return bad("gather table has the wrong size");
        uint32_t mx = 0;
        for (uint32_t v : w.idx) mx = std::max(mx, v);
        if (w.x_base_off + (uint64_t)mx + pitch > canvas_elems) return bad("a gather offset leaves the canvas");
    }
    if (!w.shifts.empty()) {
        const size_t want = w.run_rows.empty() ? (size_t)groups * w.fan_in : w.run_rows.size();
        if (w.shifts.size() != want) return bad("shift table has the wrong size");
        const uint32_t flen = w.frame_len ? w.frame_len : pitch;
        if (pitch % flen) return bad("frame length must divide the row pitch");
    }
    if (!w.bias.empty() && w.bias.size() != w.cout) return bad("bias has the wrong size");
    if (!w.cout_map.empty()) {
        if (w.cout_map.size() != w.cout) return bad("row map has the wrong size");
        for (uint16_t m : w.cout_map)
            if (w.y_off + ((uint64_t)m + 1) * pitch > canvas_elems) return bad("row map target leaves the canvas");
    }
    if (w.act < 0 || w.act > ACT_GELU) return bad("unknown activation");
    return true;
}

GatherPlan analyze_gather(const HostWave &w, uint32_t pitch, uint64_t canvas_elems) {
    GatherPlan gp;
    uint32_t groups = w.cout / w.group;
    const uint64_t total_rows = canvas_elems / pitch;
    // Groups whose gather lists are all identical (every dense layer) behave like one big group.
    if (groups > 1u) {
        bool same = true;
        const size_t per_i = w.run_rows.empty() ? w.fan_in : w.run_rows.size() / groups;
        const auto &tab = w.run_rows.empty() ? w.idx : w.run_rows;
        for (uint32_t g = 1; g < groups && same; ++g) {
            same = std::equal(tab.begin(), tab.begin() + per_i, tab.begin() + g * per_i);
            if (same && !w.shifts.empty()) same = std::equal(w.shifts.begin(), w.shifts.begin() + per_i, w.shifts.begin() + g * per_i);
        }
        if (same) { groups = 1u; gp.shared_by_all = true; }
    }
    if (!(w.group % kTileM == 0u || groups == 1u)) {
        gp.why_not = "group size is not a multiple of 128 neurons";
        gp.small_group = true;            // the run table below still serves the general kernels
    }
    struct Run { uint32_t row, len, shift; };
    std::vector<std::vector<Run>> runs(groups);
    if (!w.run_rows.empty()) {
        const uint32_t per = w.fan_in / w.run_len;
        for (uint32_t g = 0; g < groups; ++g)
            for (uint32_t r = 0; r < per; ++r)
                runs[g].push_back({w.run_rows[(size_t)g * per + r], w.run_len, w.shifts.empty() ? 0u : w.shifts[(size_t)g * per + r]});
    } else {
        for (uint32_t g = 0; g < groups; ++g) {
            const uint32_t *row_idx = w.idx.data() + (size_t)g * w.fan_in;
            const uint8_t *row_sh = w.shifts.empty() ? nullptr : w.shifts.data() + (size_t)g * w.fan_in;
            auto &rg = runs[g];
            for (uint32_t s = 0; s < w.fan_in; ++s) {
                uint64_t row;
                uint32_t sh = 0;
                if (s < w.fan_in_raw) {
                    const uint64_t e = w.x_base_off + row_idx[s];
                    if (e % pitch) { gp.why_not = "gather offsets are not row aligned (token / pixel shift given as raw offsets)"; return gp; }
                    row = e / pitch;
                    sh = row_sh ? row_sh[s] : 0u;
                } else {
                    // zero-weight padding slot: free to continue the previous run while it stays inside the canvas
                    row = (!rg.empty() && (uint64_t)rg.back().row + rg.back().len < total_rows) ? (uint64_t)rg.back().row + rg.back().len : 0;
                    sh = rg.empty() ? 0u : rg.back().shift;
                }
                if (!rg.empty() && (uint64_t)rg.back().row + rg.back().len == row && rg.back().shift == sh) ++rg.back().len;
                else rg.push_back({(uint32_t)row, 1u, sh});
            }
        }
    }
    for (auto &rg : runs)
        for (auto &r : rg) gp.max_shift = std::max(gp.max_shift, r.shift);
    uint32_t h = 64;
    for (auto &rg : runs)
        for (auto &r : rg)
            while (h >= 8 && r.len % h) h >>= 1;
    const uint32_t tail = (kStageK - w.fan_in % kStageK) % kStageK;
    while (h >= 8 && tail % h) h >>= 1;
    if (h < 8) {
        // scattered rows (the reference's own benchmark tables: one sorted random row per synapse): one table entry per
        // synapse; the streaming tcgen05 kernel fetches them row by row, the general kernels read the same table
        if (gp.max_shift > 0) { gp.why_not = "shifted runs must be made of whole 8-row blocks"; return gp; }
        h = 1;
    }
    if (gp.max_shift > 0 && h < 16 && !gp.small_group) { gp.why_not = "shifted runs must be made of whole 16-row blocks"; return gp; }
    if (gp.max_shift > 8) { gp.why_not = "token shifts above 8 columns"; return gp; }
    if (total_rows > kBoxRowMask) { gp.why_not = "canvas has more than 2^28 rows"; return gp; }
    gp.box_h = h;
    gp.boxes_per_group = (w.fan_in + tail) / h;
    gp.box_rows.reserve((size_t)groups * gp.boxes_per_group);
    for (auto &rg : runs) {
        for (auto &r : rg)
            for (uint32_t o = 0; o < r.len; o += h) gp.box_rows.push_back((r.row + o) | (r.shift << 28));
        for (uint32_t o = 0; o < tail; o += h) gp.box_rows.push_back(0u);
    }
    for (uint32_t r : gp.box_rows)
        if ((uint64_t)(r & kBoxRowMask) + h > total_rows) { gp.why_not = "a run leaves the canvas"; gp.box_rows.clear(); return gp; }
    gp.box_ok = true;
    return gp;
}

void compute_peer_slack(const uint64_t *hulls, int world, size_t launches, uint32_t *out_slack) {
    struct H { uint64_t rlo, rhi, wlo, whi; };
    std::vector<H> u(launches, H{~0ull, 0, ~0ull, 0});
    for (int r = 0; r < world; ++r)
        for (size_t n = 0; n < launches; ++n) {
            const uint64_t *h = hulls + ((size_t)r * launches + n) * 4u;
            if (h[0] < h[1]) { u[n].rlo = std::min(u[n].rlo, h[0]); u[n].rhi = std::max(u[n].rhi, h[1]); }
            if (h[2] < h[3]) { u[n].wlo = std::min(u[n].wlo, h[2]); u[n].whi = std::max(u[n].whi, h[3]); }
        }
    auto overlap = [](uint64_t a0, uint64_t a1, uint64_t b0, uint64_t b1) { return a0 < a1 && b0 < b1 && a0 < b1 && b0 < a1; };
    for (size_t n = 0; n < launches; ++n) {
        uint32_t slack = 0;
        for (size_t back = 1; back <= launches; ++back, ++slack) {          // launch n - back, cyclically
            const H &m = u[(n + launches - back % launches) % launches], &c = u[n];
            if (overlap(m.wlo, m.whi, c.rlo, c.rhi) || overlap(m.rlo, m.rhi, c.wlo, c.whi) || overlap(m.wlo, m.whi, c.wlo, c.whi)) break;
        }
        out_slack[n] = std::min<uint32_t>(slack, launches ? (uint32_t)launches - 1u : 0u);
    }
}

// tcgen05 shared-memory operand descriptors (64-bit): start address >> 4 in bits 0-13, leading-dimension
// byte offset >> 4 in bits 16-29, stride-dimension byte offset >> 4 in bits 32-45, descriptor version 1 in
// bits 46-47, layout type in bits 61-63 (2 = 128-byte swizzle).
static uint64_t smem_desc_bits(uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) |
           ((uint64_t)layout << 61);
}

UmmaDesc make_umma_desc(uint32_t n_tile) {
    UmmaDesc d;
    d.n_tile = n_tile;
    // A = weights, K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart; a K=16 step
    // moves 32 bytes along the row.
    d.a_base = smem_desc_bits(16, 1024, 2);
    d.a_k_step = 32 >> 4;
    // B = substrate tile, MN-major (columns contiguous), 128-byte swizzle: each synapse row is 128 bytes (64
    // columns); 8-row groups 1024 bytes apart (stride dimension = K); further 64-column blocks 8 KiB apart
    // (leading dimension = N). A K=16 step moves 16 rows = 2048 bytes.
    d.b_base = smem_desc_bits(kStageK * 128u, 1024, 2);
    d.b_k_step = 2048 >> 4;
    // instruction descriptor: FP32 accumulate (bit 4), A/B FP16 (0), A K-major (bit 15 = 0), B MN-major
    // (bit 16 = 1), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
    d.idesc = (1u << 4) | (1u << 16) | ((n_tile >> 3) << 17) | ((kTileM >> 4) << 24);
    d.wait_cycles = 4000000000ull;     // about two seconds at boost clock
    if (const char *e = std::getenv("K44B_ROWS_MODE")) { const int m = std::atoi(e); if (m == 1 || m == 2) d.rows_mode = (uint32_t)m; }
    if (const char *e = std::getenv("K44B_WAIT_MS")) {     // bound of every in-kernel wait, in milliseconds at ~2 GHz
        const long ms = std::atol(e);
        if (ms > 0 && ms <= 60000) d.wait_cycles = (unsigned long long)ms * 2000000ull;
    }
    return d;
}

// ---------------------------------------------------------------------------------------------------
// executor
// ---------------------------------------------------------------------------------------------------
bool Executor::check(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    err = std::string(what) + ": " + cudaGetErrorString(e);
    return false;
}

void Executor::release() {
    if (device_ >= 0) cudaSetDevice(device_);
    for (auto &w : waves_) {
        cudaFree(w.d_weights); cudaFree(w.d_gather); cudaFree(w.d_bias); cudaFree(w.d_map); cudaFree(w.d_idx_table); cudaFree(w.d_shifts); cudaFree(w.d_out_maps);
    }
    waves_.clear();
    drop_graph();
    cudaFree(d_scratch_); d_scratch_ = nullptr;
    cudaFree(d_counters_); d_counters_ = nullptr;
    scratch_tiles_ = 0;
    for (void *p : ipc_opened_) cudaIpcCloseMemHandle(p);
    ipc_opened_.clear();
    cudaFree(d_pos_); d_pos_ = nullptr;
    cudaFree(d_tokens_); d_tokens_ = nullptr;
    cudaFree(d_next_tokens_); d_next_tokens_ = nullptr;
    cudaFree(d_argmax_); d_argmax_ = nullptr; argmax_words_ = 0;
    cudaFree(d_decode_partial_); d_decode_partial_ = nullptr; decode_partial_bytes_ = 0;
    cudaFree(d_sync_); d_sync_ = nullptr;
    cudaFree(d_peers_); d_peers_ = nullptr;
    cudaFree(canvas_); canvas_ = nullptr;
    cudaFree(d_status_); d_status_ = nullptr;
    cudaFree(d_in_f32_); d_in_f32_ = nullptr;
    cudaFree(d_out_f32_); d_out_f32_ = nullptr;
    if (ev0_) { cudaEventDestroy(ev0_); ev0_ = nullptr; }
    if (copy_stream_) { cudaStreamSynchronize(copy_stream_); cudaStreamDestroy(copy_stream_); copy_stream_ = nullptr; }
    if (ev_uploaded_) { cudaEventDestroy(ev_uploaded_); ev_uploaded_ = nullptr; }
    if (ev_stage_free_) { cudaEventDestroy(ev_stage_free_); ev_stage_free_ = nullptr; }
    if (d_stage_in_) { cudaFree(d_stage_in_); d_stage_in_ = nullptr; }
    stage_pending_ = false;
    if (ev1_) { cudaEventDestroy(ev1_); ev1_ = nullptr; }
    canvas_elems_ = 0;
    is_2d_ = false;
}

bool Executor::begin(int device, uint64_t canvas_elems, uint32_t pitch, uint32_t columns, int force_path) {
    release();
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return fail("no CUDA device: this library has no CPU path");
    if (device < 0 || device >= count) return fail("device ordinal out of range");
    if (!check(cudaSetDevice(device), "cudaSetDevice")) return false;
    cudaDeviceProp prop{};
    if (!check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return false;
    if (prop.major != 10) return fail(std::string("device '") + prop.name + "' is not sm_100: kernels are built for B200 only");
    device_ = device;
    num_sms_ = prop.multiProcessorCount;
    force_path_ = force_path;
    if (const char *e = std::getenv("K44B_PDL")) pdl_ = std::atoi(e) != 0;
    if (const char *e = std::getenv("K44B_FORCE_PATH")) {
        if (!std::strcmp(e, "fma")) force_path_ = 0;
        else if (!std::strcmp(e, "umma")) force_path_ = 1;
    }
    if (pitch == 0 || pitch % 64u) return fail("row pitch must be a multiple of 64");
    if (canvas_elems == 0 || canvas_elems % 8u) return fail("canvas size must be a positive multiple of 8 elements");
    pitch_ = pitch; columns_ = columns ? columns : pitch; canvas_elems_ = canvas_elems;
    if (!check(cudaMalloc(&canvas_, canvas_elems * sizeof(__half)), "canvas allocation")) { canvas_ = nullptr; return false; }
    if (!check(cudaMemset(canvas_, 0, canvas_elems * sizeof(__half)), "canvas clear")) return false;
    if (!check(cudaMalloc(&d_status_, kStatusBytes), "status allocation")) return false;
    if (!check(cudaMemset(d_status_, 0, kStatusBytes), "status clear")) return false;
    if (!check(cudaEventCreate(&ev0_), "event") || !check(cudaEventCreate(&ev1_), "event")) return false;
    if (!check(umma_kernel_setup(), "kernel attribute setup") || !check(mma_kernel_setup(), "kernel attribute setup")) return false;
    return true;
}

// Tensor map over `rows` rows of `pitch_` FP16 elements starting at `base` (a device address valid on this GPU: the own
// canvas or a peer's mapping), boxes of box_cols x box_rows.
bool Executor::encode_map(CUtensorMap *map, void *base, uint64_t rows, uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn)
            return fail("cuTensorMapEncodeTiled is not available from the driver");
        encode = (EncodeFn)fn;
    }
    const cuuint64_t dims[2] = {pitch_, rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch_ * 2u};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return true;
}

bool Executor::make_tensor_map(DeviceWave &dw, uint32_t box_cols, bool swizzle128) {
    return encode_map(&dw.tmap, canvas_, canvas_elems_ / pitch_, box_cols, dw.args.box_h, swizzle128);
}

// Output tensor maps of a wave on the streaming tcgen05 kernel: entry 0 covers the wave's rows in this rank's canvas,
// entries 1.. the same rows in the peers' canvases (`peer_canvases`, n of them; may be null).
bool Executor::upload_out_maps(DeviceWave &dw, void *const *peer_canvases, uint32_t n) {
    std::vector<CUtensorMap> maps(1u + n);
    const uint32_t box_rows = std::min<uint32_t>(kTileM, dw.args.cout);
    if (!encode_map(&maps[0], canvas_ + dw.args.y_off, dw.args.cout, 64u, box_rows, true)) return false;
    for (uint32_t q = 0; q < n; ++q)
        if (!encode_map(&maps[1u + q], (__half *)peer_canvases[q] + dw.args.y_off, dw.args.cout, 64u, box_rows, true)) return false;
    if (!dw.d_out_maps && !check(cudaMalloc(&dw.d_out_maps, (1u + kMaxPeers) * sizeof(CUtensorMap)), "output tensor map allocation")) return false;
    if (!check(cudaMemcpy(dw.d_out_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice), "output tensor map upload")) return false;
    dw.args.out_maps = (const CUtensorMap *)dw.d_out_maps;
    dw.args.n_out_maps = 1u + n;
    return true;
}

int *Executor::decode_pos_ptr() {
    if (!ready()) { fail("executor not initialised"); return nullptr; }
    if (!d_pos_) {
        if (!check(cudaSetDevice(device_), "cudaSetDevice") || !check(cudaMalloc(&d_pos_, sizeof(int)), "position word allocation") ||
            !check(cudaMemset(d_pos_, 0, sizeof(int)), "position word clear"))
            return nullptr;
    }
    return d_pos_;
}

static int *alloc_words(int device, uint32_t n, std::string &err) {
    int *p = nullptr;
    if (cudaSetDevice(device) != cudaSuccess || cudaMalloc(&p, (size_t)n * sizeof(int)) != cudaSuccess || cudaMemset(p, 0, (size_t)n * sizeof(int)) != cudaSuccess) {
        err = "token buffer allocation failed";
        cudaFree(p);
        return nullptr;
    }
    return p;
}
int *Executor::tokens_ptr() {
    if (!ready()) { fail("executor not initialised"); return nullptr; }
    if (!d_tokens_) d_tokens_ = alloc_words(device_, pitch_, err);
    return d_tokens_;
}
int *Executor::next_tokens_ptr() {
    if (!ready()) { fail("executor not initialised"); return nullptr; }
    if (!d_next_tokens_) d_next_tokens_ = alloc_words(device_, pitch_, err);
    return d_next_tokens_;
}

// Element-wise / attention step: range-checked here, launched from the same command list as the waves.
bool Executor::add_aux(const HostWave &w) {
    if (!ready()) return fail("executor not initialised");
    if (d_peers_) return fail("commands cannot be added after the peers were set");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    DeviceWave dw;
    dw.name = w.name; dw.is_aux = true; dw.path = PATH_AUX;
    AuxArgs &x = dw.aux;
    x.kind = w.kind; x.canvas = canvas_; x.pitch = pitch_; x.columns = columns_;
    x.src_off = w.src_off; x.src2_off = w.src2_off; x.src3_off = w.src3_off; x.dst_off = w.y_off;
    x.rows = w.cout; x.eps = w.eps;
    x.h_q = w.h_q; x.h_kv = w.h_kv; x.head_dim = w.head_dim; x.seq_len = w.seq_len ? w.seq_len : pitch_; x.max_seq = w.max_seq;
    x.llama3 = w.llama3_scaling ? 1u : 0u; x.neg_log_theta = -std::log(w.rope_theta > 0.f ? w.rope_theta : 10000.0f);
    x.kcache_off = w.kcache_off; x.vcache_off = w.vcache_off;
    auto inside = [&](uint64_t off, uint64_t rows) { return off % 8u == 0u && off + rows * pitch_ <= canvas_elems_; };
    uint64_t rlo = ~0ull, rhi = 0;
    auto reads = [&](uint64_t off, uint64_t rows) { rlo = std::min(rlo, off); rhi = std::max(rhi, off + rows * pitch_); };
    switch (w.kind) {
    case AUX_RMSNORM:
        if (!w.cout || !inside(w.src_off, w.cout) || !inside(w.y_off, w.cout)) return fail("RMSNorm '" + w.name + "' leaves the canvas");
        if (!w.bias.empty()) {
            if (w.bias.size() != w.cout) return fail("RMSNorm '" + w.name + "': gamma has the wrong length");
            if (!check(cudaMalloc(&dw.d_bias, w.bias.size() * 2), "gamma allocation") ||
                !check(cudaMemcpy(dw.d_bias, w.bias.data(), w.bias.size() * 2, cudaMemcpyHostToDevice), "gamma upload")) return false;
            x.gamma = (const __half *)dw.d_bias;
        }
        reads(w.src_off, w.cout);
        dw.write_lo = w.y_off; dw.write_hi = w.y_off + (uint64_t)w.cout * pitch_;
        break;
    case AUX_SWIGLU:
        if (!w.cout || !inside(w.src_off, w.cout) || !inside(w.src2_off, w.cout) || !inside(w.y_off, w.cout)) return fail("SwiGLU '" + w.name + "' leaves the canvas");
        reads(w.src_off, w.cout); reads(w.src2_off, w.cout);
        dw.write_lo = w.y_off; dw.write_hi = w.y_off + (uint64_t)w.cout * pitch_;
        break;
    case AUX_ROPE_ATTN:
    case AUX_DECODE_ATTN: {
        if ((w.head_dim != 64u && w.head_dim != 128u) || !w.h_kv || !w.h_q || w.h_q % w.h_kv) return fail("attention '" + w.name + "': head_dim must be 64 or 128 and h_q a multiple of h_kv");
        const uint64_t rq = (uint64_t)w.h_q * w.head_dim, rk = (uint64_t)w.h_kv * w.head_dim;
        if (!inside(w.src_off, rq) || !inside(w.src2_off, rk) || !inside(w.src3_off, rk) || !inside(w.y_off, rq)) return fail("attention '" + w.name + "' leaves the canvas");
        if (w.kind == AUX_ROPE_ATTN) {
            if (pitch_ % 32u || x.seq_len % 32u) return fail("attention '" + w.name + "': sequences must be multiples of 32 columns");
        } else {
            if (!w.max_seq || w.kcache_off % 8u || w.vcache_off % 8u || w.kcache_off + rk * w.max_seq * pitch_ > canvas_elems_ ||
                w.vcache_off + rk * w.max_seq * pitch_ > canvas_elems_) return fail("attention '" + w.name + "': key / value cache leaves the canvas");
            { const uint32_t grp = w.h_q / w.h_kv; if (w.head_dim != 64u || !(grp == 1u || grp == 2u || grp == 4u || grp == 8u)) return fail("attention '" + w.name + "': the cache kernel supports head_dim 64 and 1, 2, 4 or 8 query heads per key / value head"); }
            if (!(x.pos_ptr = decode_pos_ptr())) return false;
            const size_t pbytes = (size_t)((w.max_seq + kDecodeChunk - 1u) / kDecodeChunk) * w.h_q * kDecodeRow * pitch_ * sizeof(float);
            if (pbytes > decode_partial_bytes_) {
                if (!check(cudaDeviceSynchronize(), "synchronise")) return false;
                cudaFree(d_decode_partial_); d_decode_partial_ = nullptr; decode_partial_bytes_ = 0;
                if (!check(cudaMalloc(&d_decode_partial_, pbytes), "attention scratch allocation")) return false;
                decode_partial_bytes_ = pbytes;
                for (auto &o : waves_) if (o.is_aux && o.aux.kind == AUX_DECODE_ATTN) o.aux.partial = d_decode_partial_;
            }
            x.partial = d_decode_partial_;
            reads(w.kcache_off, rk * w.max_seq); reads(w.vcache_off, rk * w.max_seq);
        }
        reads(w.src_off, rq); reads(w.src2_off, rk); reads(w.src3_off, rk);
        // q and k are rotated in place, the caches are appended to: treat everything touched as written
        dw.write_lo = std::min({w.y_off, w.src_off, w.src2_off, rlo}); dw.write_hi = std::max({w.y_off + rq * pitch_, rhi});
        break;
    }
    case AUX_EMBED:
        if (!w.cout || w.cout % 8u || !w.dev_table || !w.vocab || !inside(w.y_off, w.cout)) return fail("embedding '" + w.name + "': bad table or destination");
        x.table = (const __half *)w.dev_table; x.vocab = w.vocab;
        if (!(x.tokens = tokens_ptr())) return false;
        rlo = 0; rhi = 0;
        dw.write_lo = w.y_off; dw.write_hi = w.y_off + (uint64_t)w.cout * pitch_;
        break;
    case AUX_ARGMAX: {
        if (!w.cout || pitch_ % 64u || !inside(w.src_off, w.cout)) return fail("arg-max '" + w.name + "' leaves the canvas");
        x.advance = w.advance ? 1u : 0u; x.max_seq = w.max_seq;
        if (!(x.next_tokens = next_tokens_ptr()) || !(x.tokens = tokens_ptr())) return false;
        if (w.advance && !(x.pos_rw = decode_pos_ptr())) return false;
        const size_t words = (size_t)((w.cout + kArgmaxChunk - 1u) / kArgmaxChunk) * pitch_;
        if (words > argmax_words_) {
            if (!check(cudaDeviceSynchronize(), "synchronise")) return false;
            cudaFree(d_argmax_); d_argmax_ = nullptr; argmax_words_ = 0;
            if (!check(cudaMalloc(&d_argmax_, words * sizeof(unsigned long long)), "arg-max scratch allocation")) return false;
            argmax_words_ = words;
            for (auto &o : waves_) if (o.is_aux && o.aux.kind == AUX_ARGMAX) o.aux.argmax_scratch = d_argmax_;
        }
        x.argmax_scratch = d_argmax_;
        reads(w.src_off, w.cout);
        dw.write_lo = 0; dw.write_hi = 0;
        break;
    }
    case AUX_MAXPOOL2: case AUX_MAXPOOL5: case AUX_UPSAMPLE2: case AUX_S2D: case AUX_UPCONV_SCATTER: case AUX_HALO_CLEAR: {
        // planes of a 2-D image tensor: geometry from the plan, everything range-checked here
        const auto &gi = w.in2d, &go = w.out2d;
        x.h_in = gi.H; x.w_in = gi.W; x.wpad_in = gi.W_pad; x.cs_in = gi.ch_stride;
        x.h_out = go.H; x.w_out = go.W; x.wpad_out = go.W_pad; x.cs_out = go.ch_stride;
        x.frames = std::max(1u, go.frames);
        x.fs_in = gi.frame_stride ? gi.frame_stride : gi.ch_stride; x.fs_out = go.frame_stride ? go.frame_stride : go.ch_stride;
        if (w.kind != AUX_HALO_CLEAR && std::max(1u, gi.frames) != x.frames) return fail("image command '" + w.name + "': input and output hold different numbers of frames");
        if ((uint64_t)x.frames * x.fs_out > go.ch_stride || (w.kind != AUX_HALO_CLEAR && (uint64_t)x.frames * x.fs_in > gi.ch_stride))
            return fail("image command '" + w.name + "': the frames do not fit the channel stride");
        const uint32_t src_planes = w.kind == AUX_UPCONV_SCATTER ? 4u * w.cout : w.cout;
        const uint32_t dst_planes = w.kind == AUX_S2D ? 4u * w.cout : w.cout;
        auto plane_ok = [&](const HostWave::Geom2D &g) { return g.H && g.W && g.W_pad >= g.W + 4u && (uint64_t)(g.H + 2u) * g.W_pad <= (uint64_t)(g.frame_stride ? g.frame_stride : g.ch_stride) + 8u; };
        if (!w.cout || !plane_ok(go) || (w.kind != AUX_HALO_CLEAR && !plane_ok(gi))) return fail("image command '" + w.name + "': bad plane geometry");
        if (w.y_off + (uint64_t)dst_planes * go.ch_stride > canvas_elems_) return fail("image command '" + w.name + "' writes outside the canvas");
        if (w.kind != AUX_HALO_CLEAR && w.src_off + (uint64_t)src_planes * gi.ch_stride > canvas_elems_) return fail("image command '" + w.name + "' reads outside the canvas");
        bool shape_ok = true;
        switch (w.kind) {
        case AUX_MAXPOOL2: case AUX_S2D: shape_ok = gi.H == 2u * go.H && gi.W == 2u * go.W; break;
        case AUX_UPSAMPLE2: case AUX_UPCONV_SCATTER: shape_ok = go.H == 2u * gi.H && go.W == 2u * gi.W; break;
        case AUX_MAXPOOL5: shape_ok = gi.H == go.H && gi.W == go.W; break;
        default: break;
        }
        if (!shape_ok) return fail("image command '" + w.name + "': source and destination sizes do not fit the operation");
        if (w.kind != AUX_HALO_CLEAR) { rlo = w.src_off; rhi = w.src_off + (uint64_t)src_planes * gi.ch_stride; }
        else { rlo = 0; rhi = 0; }
        dw.write_lo = w.y_off; dw.write_hi = w.y_off + (uint64_t)dst_planes * go.ch_stride;
        break;
    }
    default: return fail("unknown command kind");
    }
    dw.read_lo = rlo; dw.read_hi = rhi;
    dw.groupable = false;
    waves_.push_back(dw);
    drop_graph();
    groups_valid_ = false;
    return true;
}

// A wave over 2-D image planes (convolution taps as element offsets relative to per-tile anchors, outputs at per-tile plane
// offsets, optionally masked by 4-element quads): always on the general kernels — the warp-level tensor path, or the FP32-FMA
// kernel when forced — whose gathers take any element alignment. The role of the reference's unaligned token-shift kernel
// for image layouts (kernels/cuda/kernel44_cuda_pack.cuh:242-264; wavec/k44_wave_executor.cu:245-255).
bool Executor::add_wave_2d(const HostWave &w) {
    auto bad = [&](const std::string &m) { return fail("wave '" + w.name + "': " + m); };
    const uint32_t tiles = (uint32_t)w.tile_off_x.size();
    if (!tiles || w.tile_off_y.size() != tiles) return bad("tile tables missing or of different lengths");
    if (w.cout == 0 || w.cout % 16u || w.group == 0 || w.cout % w.group || w.group % 16u) return bad("row count / group size must be multiples of 16");
    if (w.fan_in == 0 || w.fan_in % 8u || w.fan_in_raw > w.fan_in) return bad("bad fan-in");
    if (w.y_off % 4u || w.res_off % 4u || w.pitch2d % 4u) return bad("plane offsets must be multiples of 4 elements");
    if (!w.cout_map.empty() || !w.shifts.empty() || !w.run_rows.empty()) return bad("row maps, shift tables and run tables do not apply to image waves");
    const uint32_t groups = w.cout / w.group;
    if (w.idx.size() != (size_t)groups * w.fan_in) return bad("gather table has the wrong size");
    if (w.w_wmma.size() != (size_t)w.cout * w.fan_in) return bad("weight block has the wrong size");
    if (!w.bias.empty() && w.bias.size() != w.cout) return bad("bias has the wrong size");
    if (w.act < 0 || w.act > ACT_GELU) return bad("unknown activation");
    uint32_t max_idx = 0, max_tx = 0, max_ty = 0;
    for (uint32_t g = 0; g < groups; ++g)
        for (uint32_t k = 0; k < w.fan_in_raw; ++k) max_idx = std::max(max_idx, w.idx[(size_t)g * w.fan_in + k]);
    for (uint32_t t = 0; t < tiles; ++t) {
        max_tx = std::max(max_tx, w.tile_off_x[t]);
        max_ty = std::max(max_ty, w.tile_mask ? (w.tile_off_y[t] & 0xffffu) << 2 : w.tile_off_y[t]);
    }
    if (w.x_base_off + (uint64_t)max_tx + max_idx + 64u > canvas_elems_) return bad("a gather leaves the canvas");
    if (w.y_off + (uint64_t)(w.cout - 1u) * w.pitch2d + max_ty + 64u > canvas_elems_) return bad("output planes leave the canvas");
    if (w.has_residual && w.res_off + (uint64_t)(w.cout - 1u) * w.pitch2d + max_ty + 64u > canvas_elems_) return bad("residual planes leave the canvas");

    DeviceWave dw;
    dw.name = w.name;
    dw.synapses = (uint64_t)w.logical_cout * w.fan_in_raw;
    WaveArgs &a = dw.args;
    a.canvas = canvas_; a.canvas_elems = canvas_elems_; a.status = d_status_;
    a.y_off = w.y_off; a.res_off = w.res_off; a.x_base_off = w.x_base_off;
    a.cout = w.cout; a.group = w.group; a.fan_in = w.fan_in;
    a.num_kstages = (w.fan_in + kStageK - 1) / kStageK;
    a.pitch = w.pitch2d; a.num_col_tiles64 = tiles;
    a.act = w.act; a.has_residual = w.has_residual ? 1 : 0;
    a.gather_mode = GATHER_IDX;
    a.tile_mask = w.tile_mask ? 1u : 0u;
    const uint32_t mtiles = (w.cout + kTileM - 1) / kTileM;
    dw.weight_bytes = (uint64_t)mtiles * a.num_kstages * kStageWBytes;
    void *stage = nullptr;
    bool ok = check(cudaMalloc(&dw.d_weights, dw.weight_bytes), "weight allocation") &&
              check(cudaMalloc(&stage, w.w_wmma.size() * 2), "staging allocation") &&
              check(cudaMemcpy(stage, w.w_wmma.data(), w.w_wmma.size() * 2, cudaMemcpyHostToDevice), "weight upload") &&
              check(launch_repack_wmma_to_tiled((const uint4 *)stage, (uint4 *)dw.d_weights, w.cout, w.fan_in, nullptr), "weight repack") &&
              check(cudaDeviceSynchronize(), "weight repack");
    cudaFree(stage);
    a.w_tiles = (const uint4 *)dw.d_weights;
    // gather table followed by the two tile tables in one allocation
    std::vector<uint32_t> tab(w.idx);
    tab.insert(tab.end(), w.tile_off_x.begin(), w.tile_off_x.end());
    tab.insert(tab.end(), w.tile_off_y.begin(), w.tile_off_y.end());
    ok = ok && check(cudaMalloc(&dw.d_gather, tab.size() * 4), "table allocation") &&
         check(cudaMemcpy(dw.d_gather, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice), "table upload");
    a.gather = (const uint32_t *)dw.d_gather;
    a.tile_off_x = a.gather + w.idx.size();
    a.tile_off_y = a.tile_off_x + tiles;
    if (ok && !w.bias.empty() && w.has_bias) {
        ok = check(cudaMalloc(&dw.d_bias, w.bias.size() * 2), "bias allocation") &&
             check(cudaMemcpy(dw.d_bias, w.bias.data(), w.bias.size() * 2, cudaMemcpyHostToDevice), "bias upload");
        a.bias = (const __half *)dw.d_bias;
    }
    if (!ok) { cudaFree(dw.d_weights); cudaFree(dw.d_gather); cudaFree(dw.d_bias); return false; }
    dw.path = force_path_ == 0 ? PATH_FMA : PATH_MMA;
    dw.fma_reason = "image planes (element-granular tap offsets, per-tile anchors)";
    dw.write_lo = w.y_off; dw.write_hi = w.y_off + (uint64_t)w.cout * w.pitch2d;
    dw.read_lo = w.x_base_off; dw.read_hi = std::min<uint64_t>(canvas_elems_, w.x_base_off + (uint64_t)max_tx + max_idx + 64u);
    if (w.has_residual) { dw.read_lo = std::min(dw.read_lo, w.res_off); dw.read_hi = std::max(dw.read_hi, w.res_off + (uint64_t)w.cout * w.pitch2d); }
    dw.groupable = false;
    peer_slack_.clear();
    waves_.push_back(dw);
    drop_graph();
    groups_valid_ = false;
    return true;
}

bool Executor::add_wave(const HostWave &w) {
    if (w.kind != 0) return add_aux(w);
    if (!ready()) return fail("executor not initialised");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    if (d_peers_) return fail("waves cannot be added after the peers were set");
    if (w.pitch2d) return add_wave_2d(w);
    const uint32_t tiles64 = pitch_ / 64u;
    if (!validate_wave(w, pitch_, tiles64, canvas_elems_, err)) return false;
    if (w.w_wmma.empty() && !w.dev_weights_rowmajor) return fail("wave '" + w.name + "' has no weights");
    if (!w.w_wmma.empty() && w.w_wmma.size() != (size_t)w.cout * w.fan_in) return fail("wave '" + w.name + "': weight block has the wrong size");
    // padding slots must carry zero weights (the packer is free to point them at any row)
    if (!w.w_wmma.empty() && w.fan_in_raw < w.fan_in) {
        for (uint32_t j = 0; j < w.cout; ++j)
            for (uint32_t s = w.fan_in_raw; s < w.fan_in; ++s)
                if (w.w_wmma[wmma_vec_index(j, s >> 3, w.fan_in) * 8u + (s & 7u)] & 0x7fffu)
                    return fail("wave '" + w.name + "': non-zero weight in a padding slot");
    }

    DeviceWave dw;
    dw.name = w.name;
    dw.synapses = (uint64_t)w.logical_cout * w.fan_in_raw;
    WaveArgs &a = dw.args;
    a.canvas = canvas_; a.canvas_elems = canvas_elems_; a.status = d_status_;
    if (d_peers_) return fail("waves cannot be added after the peers were set");
    a.y_off = w.y_off; a.res_off = w.res_off; a.x_base_off = w.x_base_off;
    a.cout = w.cout; a.group = w.group; a.fan_in = w.fan_in;
    a.num_kstages = (w.fan_in + kStageK - 1) / kStageK;
    a.pitch = pitch_; a.num_col_tiles64 = tiles64;
    a.act = w.act; a.has_residual = w.has_residual ? 1 : 0;
    const uint32_t groups = w.cout / w.group;

    // ---- weights: container order or device row-major -> tiled ----
    const uint32_t mtiles = (w.cout + kTileM - 1) / kTileM;
    dw.weight_bytes = (uint64_t)mtiles * a.num_kstages * kStageWBytes;
    if (!check(cudaMalloc(&dw.d_weights, dw.weight_bytes), "weight allocation")) return false;
    bool ok = true;
    if (w.dev_weights_rowmajor) {
        ok = check(launch_repack_rowmajor_to_tiled((const uint4 *)w.dev_weights_rowmajor, (uint4 *)dw.d_weights, w.cout, w.fan_in, nullptr), "weight repack") &&
             check(cudaDeviceSynchronize(), "weight repack");   // the caller may reuse its buffer on return
    } else {
        void *stage = nullptr;
        const size_t bytes = w.w_wmma.size() * 2;
        ok = check(cudaMalloc(&stage, bytes), "staging allocation") &&
             check(cudaMemcpy(stage, w.w_wmma.data(), bytes, cudaMemcpyHostToDevice), "weight upload") &&
             check(launch_repack_wmma_to_tiled((const uint4 *)stage, (uint4 *)dw.d_weights, w.cout, w.fan_in, nullptr), "weight repack") &&
             check(cudaDeviceSynchronize(), "weight repack");
        cudaFree(stage);
    }
    a.w_tiles = (const uint4 *)dw.d_weights;

    // ---- gather tables ----
    GatherPlan gp;
    if (ok) gp = analyze_gather(w, pitch_, canvas_elems_);
    if (ok && gp.box_ok && gp.small_group) {
        // runs of whole boxes, but groups below 128 neurons: the general kernels read the run table as it is
        const size_t bytes = gp.box_rows.size() * 4;
        ok = check(cudaMalloc(&dw.d_gather, bytes), "run table allocation") &&
             check(cudaMemcpy(dw.d_gather, gp.box_rows.data(), bytes, cudaMemcpyHostToDevice), "run table upload");
        a.gather = (const uint32_t *)dw.d_gather;
        a.gather_mode = GATHER_BOX;
        a.box_h = gp.box_h; a.boxes_per_group = gp.boxes_per_group;
        a.x_base_off = 0;                 // box rows are absolute canvas rows
        dw.fma_reason = gp.why_not;
    } else if (ok && gp.box_ok) {
        const size_t bytes = gp.box_rows.size() * 4;
        ok = check(cudaMalloc(&dw.d_gather, bytes), "run table allocation") &&
             check(cudaMemcpy(dw.d_gather, gp.box_rows.data(), bytes, cudaMemcpyHostToDevice), "run table upload");
        a.gather = (const uint32_t *)dw.d_gather;
        a.gather_mode = GATHER_BOX;
        a.box_h = gp.box_h; a.boxes_per_group = gp.boxes_per_group;
        a.x_base_off = 0;                 // box rows are absolute canvas rows
        a.mtiles_per_group = (groups == 1u || gp.shared_by_all) ? (w.cout + kTileM - 1) / kTileM : std::max(1u, w.group / kTileM);
        if (gp.shared_by_all) a.group = w.cout;   // the run table holds a single list
        dw.umma_capable = true;
    } else if (ok) {
        dw.fma_reason = gp.why_not;
        if (w.idx.empty()) { ok = fail("wave '" + w.name + "': run table unusable (" + gp.why_not + ") and no index table given"); }
        else {
            const size_t bytes = w.idx.size() * 4;
            ok = check(cudaMalloc(&dw.d_gather, bytes), "index table allocation") &&
                 check(cudaMemcpy(dw.d_gather, w.idx.data(), bytes, cudaMemcpyHostToDevice), "index table upload");
            a.gather = (const uint32_t *)dw.d_gather;
            a.gather_mode = GATHER_IDX;
            if (ok && !w.shifts.empty()) {
                ok = check(cudaMalloc(&dw.d_shifts, w.shifts.size()), "shift table allocation") &&
                     check(cudaMemcpy(dw.d_shifts, w.shifts.data(), w.shifts.size(), cudaMemcpyHostToDevice), "shift table upload");
                a.shifts = (const uint8_t *)dw.d_shifts;
            }
        }
    }
    a.frame_len = w.frame_len;
    a.has_shift = w.shifts.empty() ? 0u : 1u;
    if (ok && !w.bias.empty() && w.has_bias) {
        ok = check(cudaMalloc(&dw.d_bias, w.bias.size() * 2), "bias allocation") &&
             check(cudaMemcpy(dw.d_bias, w.bias.data(), w.bias.size() * 2, cudaMemcpyHostToDevice), "bias upload");
        a.bias = (const __half *)dw.d_bias;
    }
    if (ok && !w.cout_map.empty()) {
        ok = check(cudaMalloc(&dw.d_map, w.cout_map.size() * 2), "row map allocation") &&
             check(cudaMemcpy(dw.d_map, w.cout_map.data(), w.cout_map.size() * 2, cudaMemcpyHostToDevice), "row map upload");
        a.cout_map = (const uint16_t *)dw.d_map;
    }
    // ---- path and tile shape ----
    if (ok) {
        // A shift of 1..7 columns can be neither an operand start address nor an accumulator column offset
        // (tcgen05.mma rejects the latter with a misaligned-address fault).
        // Token-shifted runs take the aligner kernel: its extra warps realign the shifted rows in registers on the way
        // into the operand stage. It needs frames that are whole column tiles; otherwise the wave stays on FMA.
        if (gp.max_shift > 0) {
            const uint32_t flen = w.frame_len ? w.frame_len : pitch_;
            bool allow = dw.umma_capable && flen % 64u == 0u;
            if (const char *e = std::getenv("K44B_SHIFT_UMMA")) allow = allow && std::atoi(e) != 0;
            if (!allow) { dw.umma_capable = false; dw.fma_reason = flen % 64u ? "token-shifted runs with frames that are not whole column tiles" : "token-shifted runs"; }
            else dw.use_shift = true;
        }
        // scattered single rows are fetched by the streaming tcgen05 kernel only; a wave with fewer tiles than SMs (which would
        // take the small-wave kernel) stays on the warp-level tensor path
        if (dw.umma_capable && gp.box_h == 1u && (uint64_t)mtiles * tiles64 < (uint64_t)num_sms_) {
            dw.umma_capable = false;
            dw.fma_reason = "scattered rows in a wave with fewer 128-neuron tiles than SMs";
        }
        // waves the tcgen05 kernels cannot take run on the warp-level tensor path; the FP32-FMA kernel only when asked for
        dw.path = force_path_ == 0 ? PATH_FMA : (dw.umma_capable ? PATH_UMMA : PATH_MMA);
        if (const char *e = std::getenv("K44B_GENERAL_MMA")) if (dw.path == PATH_MMA && std::atoi(e) == 0) dw.path = PATH_FMA;
        if (dw.path == PATH_UMMA && dw.use_shift) {
            const uint32_t flen = w.frame_len ? w.frame_len : pitch_;
            uint32_t n_tile = 64;
            for (uint32_t cand : {256u, 128u})
                if (tiles64 % (cand / 64u) == 0u && flen % cand == 0u && (uint64_t)mtiles * (tiles64 / (cand / 64u)) >= (uint64_t)num_sms_) { n_tile = cand; break; }
            if (const char *e = std::getenv("K44B_N_TILE")) {
                const uint32_t v = (uint32_t)std::atoi(e);
                if ((v == 64 || v == 128 || v == 256) && tiles64 % (v / 64u) == 0u && flen % v == 0u) n_tile = v;
            }
            a.k_splits = 1; a.kstages_per_split = a.num_kstages;
            dw.desc = make_umma_desc(n_tile);
            // fan-in up to 512: the weight tile of a work item stays in tensor memory (tiles of 128 columns), which takes the
            // weights out of the shared-memory traffic that bounds this kernel
            a.gather_mode = GATHER_BOX; a.box_h = gp.box_h;
            bool ws = n_tile >= 128u && flen % 128u == 0u && shift_ws_supported(a) && (uint64_t)mtiles * (tiles64 / 2u) >= (uint64_t)num_sms_;
            if (const char *e = std::getenv("K44B_SHIFT_WS")) {       // 0: never, 2: whenever the wave qualifies, however few tiles it has
                const int v = std::atoi(e);
                ws = v == 2 ? (flen % 128u == 0u && shift_ws_supported(a)) : (ws && v != 0);
            }
            if (ws) {
                dw.desc = make_umma_desc(128u);
                dw.desc.ws_chunk = shift_ws_chunk(mtiles, tiles64 / 2u, (uint32_t)num_sms_);
                if (const char *e = std::getenv("K44B_WS_CHUNK")) { const int v = std::atoi(e); if (v > 0) dw.desc.ws_chunk = (uint32_t)v; }
                if (const char *e = std::getenv("K44B_WS_GROUPS")) { const int v = std::atoi(e); if (v >= 1 && v <= 2) dw.desc.ws_groups = (uint32_t)v; }
                n_tile = 128u;
            }
            ok = make_tensor_map(dw, std::min(n_tile, 128u) + 8u, false);   // aligned windows of up to 128 columns plus the 8 to their left, as plain rows
        } else if (dw.path == PATH_UMMA) {
            uint32_t n_tile = 64;
            for (uint32_t cand : {256u, 128u})
                if (tiles64 % (cand / 64u) == 0u && (uint64_t)mtiles * (tiles64 / (cand / 64u)) >= (uint64_t)num_sms_) { n_tile = cand; break; }
            if (const char *e = std::getenv("K44B_N_TILE")) {
                const uint32_t v = (uint32_t)std::atoi(e);
                if ((v == 64 || v == 128 || v == 256) && tiles64 % (v / 64u) == 0u) n_tile = v;
            }
            // Small waves (fewer tiles than SMs): 64-column tiles, two CTAs per SM, and the fan-in cut into
            // K splits so that every SM streams a share of the weights.
            uint32_t splits = 1;
            bool small = (uint64_t)mtiles * (tiles64 / (n_tile / 64u)) < (uint64_t)num_sms_;
            if (const char *e = std::getenv("K44B_SMALL_WAVE")) small = std::atoi(e) != 0;
            if (gp.box_h == 1u) small = false;
            bool cluster = false;
            if (small) {
                n_tile = 64;
                const uint32_t tiles = mtiles * tiles64, cap = 2u * (uint32_t)num_sms_;
                splits = std::max(1u, std::min(cap / tiles, a.num_kstages / 2u));   // all items resident at once: no second round
                // preferred: the splits of a tile form a thread-block cluster (<= 8 CTAs, one CTA per SM) and add their
                // partial sums through distributed shared memory instead of global scratch
                cluster = tiles <= cap;
                if (const char *e = std::getenv("K44B_CLUSTER")) cluster = cluster && std::atoi(e) != 0;
                const char *es = std::getenv("K44B_SPLITS");
                if (es) splits = std::max(1u, std::min((uint32_t)std::atoi(es), a.num_kstages));
                if (cluster) {
                    uint32_t s2 = 8;           // portable cluster size; 16 is accepted when forced but lost to barrier and placement cost
                    while (s2 > 1 && (s2 * tiles > cap || s2 * 2u > a.num_kstages)) s2 >>= 1;   // <= two CTAs per SM
                    if (es) { s2 = 1; while (s2 * 2u <= std::min(splits, 16u)) s2 <<= 1; }
                    splits = s2;
                }
            }
            a.kstages_per_split = (a.num_kstages + splits - 1) / splits;
            a.k_splits = cluster ? splits : (a.num_kstages + a.kstages_per_split - 1) / a.kstages_per_split;
            dw.use_cluster = cluster;
            dw.desc = make_umma_desc(n_tile);
            dw.desc.small_wave = small ? 1u : 0u;
            if (a.k_splits > 1 && !cluster) ok = reserve_scratch((size_t)mtiles * tiles64);
            ok = ok && make_tensor_map(dw, 64u, true);
            // streaming waves without an output-row map write their tiles with tensor copies out of shared memory
            bool tile_copies = !small && w.cout_map.empty();
            if (const char *e = std::getenv("K44B_TILE_COPIES")) tile_copies = tile_copies && std::atoi(e) != 0;
            if (ok && tile_copies) ok = upload_out_maps(dw, nullptr, 0);
            // Tensor-bound waves (256-column tiles) whose neuron groups span an even number of 128-neuron blocks run tiles of
            // 256 neurons: two blocks share one gathered operand, which halves the operand bytes each flop pulls through L2.
            // Needs enough such tiles to fill the GPU and the tile-copy epilogue.
            {
                bool two = ok && tile_copies && n_tile == 256u && a.k_splits == 1u && (a.mtiles_per_group % 2u) == 0u &&
                      (uint64_t)((mtiles + 1u) / 2u) * (tiles64 / 4u) >= (uint64_t)num_sms_ && !(gp.box_h == 1u && dw.desc.rows_mode == 2u);
                // preferred for such waves: the two blocks on a pair of CTAs (M = 256 MMAs), see k44_pair_kernel.cu
                bool pair = two && (mtiles % 2u) == 0u && (gp.box_h == 1u || 2u * (kStageK / gp.box_h) <= 32u);   // (boxes: one producer lane per box)
                // (measured, reference-benchmark shapes: pairs 111 us against 127 us per pass for run tables when the GPU is not held
                // back by its power cap, the same ~0.17 ms once it is; for scattered rows the pair's extra hop — CTA 1's copies are
                // passed on to CTA 0's barrier — costs more than the halved fetch saves, so those stay on one CTA)
                if (const char *e = std::getenv("K44B_PAIR")) pair = pair && std::atoi(e) != 0; else pair = pair && gp.box_h != 1u;
                if (const char *e = std::getenv("K44B_M_BLOCKS")) two = two && std::atoi(e) == 2; else two = false;   // two blocks on one CTA: measured no gain, on request only
                if (pair) {
                    two = false;
                    dw.desc.pair = 1u;
                    dw.desc.idesc = (1u << 4) | (1u << 16) | ((256u >> 3) << 17) | ((256u >> 4) << 24);   // M = 256, N = 256
                    // the packed weights as a 2-D tensor: rows of 128 bytes (64 halves), one 128-row box = one 16 KiB block
                    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
                    void *fn = nullptr;
                    cudaDriverEntryPointQueryResult q;
                    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) ok = fail("cuTensorMapEncodeTiled is not available from the driver");
                    if (ok) {
                        const cuuint64_t dims[2] = {64u, (cuuint64_t)mtiles * a.num_kstages * kTileM};
                        const cuuint64_t strides[1] = {128u};
                        const cuuint32_t box[2] = {64u, kTileM};
                        const cuuint32_t estr[2] = {1u, 1u};
                        const CUresult r = ((EncodeFn)fn)(&dw.wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, dw.d_weights, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                        if (r != CUDA_SUCCESS) ok = fail("cuTensorMapEncodeTiled (weights) failed with code " + std::to_string((int)r));
                    }
                }
                dw.desc.m_blocks = two ? 2u : 1u;
            }
        }
    }
    if (!ok) {
        cudaFree(dw.d_weights); cudaFree(dw.d_gather); cudaFree(dw.d_bias); cudaFree(dw.d_map); cudaFree(dw.d_shifts); cudaFree(dw.d_out_maps);
        return false;
    }
    // canvas intervals for the scheduler's independence test
    dw.write_lo = w.y_off; dw.write_hi = w.y_off + (uint64_t)w.cout * pitch_;
    uint64_t lo = ~0ull, hi = 0;
    if (gp.box_ok) {
        for (uint32_t e : gp.box_rows) { const uint64_t r = e & kBoxRowMask; lo = std::min(lo, r * pitch_); hi = std::max(hi, (r + gp.box_h) * pitch_); }
    } else {
        for (uint32_t v : w.idx) { lo = std::min(lo, w.x_base_off + v); hi = std::max(hi, w.x_base_off + v + pitch_); }
        if (lo >= 8) lo -= 8;                       // shifted taps read a few columns to the left
    }
    if (w.has_residual) { lo = std::min(lo, w.res_off); hi = std::max(hi, w.res_off + (uint64_t)w.cout * pitch_); }
    dw.read_lo = lo; dw.read_hi = hi;
    // A wave must not gather rows it writes: CTAs of one launch would race, and in a neuron-sharded plan a peer's stores
    // of launch n would land in rows this rank's launch n still reads (residual rows may equal the output rows: each
    // element is read and written by the same thread).
    {
        uint64_t wlo = dw.write_lo, whi = dw.write_hi;
        if (!w.cout_map.empty()) { uint32_t mx = 0; for (uint16_t m : w.cout_map) mx = std::max<uint32_t>(mx, m); whi = w.y_off + ((uint64_t)mx + 1) * pitch_; dw.write_hi = std::max(dw.write_hi, whi); }
        bool clash = false;
        // (checked on the caller's tables: zero-weight padding slots, which the packer points wherever it likes, do not count)
        if (!w.run_rows.empty()) {
            for (uint32_t r : w.run_rows) { const uint64_t r0 = (uint64_t)r * pitch_; if (r0 < whi && wlo < r0 + (uint64_t)w.run_len * pitch_) { clash = true; break; } }
        } else {
            for (uint32_t g = 0; g < groups && !clash; ++g)
                for (uint32_t sidx = 0; sidx < w.fan_in_raw; ++sidx) {
                    const uint64_t e0 = w.x_base_off + w.idx[(size_t)g * w.fan_in + sidx];
                    if ((e0 >= 8 ? e0 - 8 : 0) < whi && wlo < e0 + pitch_) { clash = true; break; }
                }
        }
        if (clash) {
            cudaFree(dw.d_weights); cudaFree(dw.d_gather); cudaFree(dw.d_bias); cudaFree(dw.d_map); cudaFree(dw.d_shifts); cudaFree(dw.d_out_maps);
            return fail("wave '" + w.name + "' gathers rows that it writes (a wave cannot run in place)");
        }
    }
    dw.groupable = dw.path == PATH_UMMA && dw.use_cluster && w.cout_map.empty();
    peer_slack_.clear();
    waves_.push_back(dw);
    drop_graph();
    groups_valid_ = false;
    return true;
}

void Executor::set_io(uint64_t in_off, uint32_t in_c, uint64_t out_off, uint32_t out_c, uint32_t width) {
    in_off_ = in_off; in_c_ = in_c; out_off_ = out_off; out_c_ = out_c; io_width_ = width;
}

bool Executor::init(const HostPlan &plan, int device, int force_path) {
    // (an image plan has no plan-wide row pitch: every wave carries its tensor's plane stride; 64 stands in for the checks)
    if (!begin(device, plan.canvas_elems, plan.is_2d ? 64u : plan.layout.channel_stride, plan.is_2d ? 64u : plan.layout.width, force_path)) return false;
    is_2d_ = plan.is_2d; in2d_ = plan.in2d; out2d_ = plan.out2d;
    for (const auto &w : plan.waves)
        if (!add_wave(w)) { std::string keep = err; release(); err = keep; return false; }
    set_io(plan.input_off, plan.input_c, plan.output_off, plan.logical_output_c ? plan.logical_output_c : plan.output_c, plan.layout.width);
    if (is_2d_) {
        if ((uint64_t)in_off_ + (uint64_t)in_c_ * in2d_.ch_stride > canvas_elems_ || (uint64_t)out_off_ + (uint64_t)out_c_ * out2d_.ch_stride > canvas_elems_) {
            release();
            return fail("plan input / output planes leave the canvas");
        }
        return true;
    }
    if ((uint64_t)in_off_ + (uint64_t)in_c_ * pitch_ > canvas_elems_ || (uint64_t)out_off_ + (uint64_t)out_c_ * pitch_ > canvas_elems_) {
        release();
        return fail("plan input / output region leaves the canvas");
    }
    return true;
}

// Split-K partial sums of every wave meet in one shared FP32 scratch area (waves run one after another).
// Both the scratch and the per-tile arrival counters are zero between launches: the finishing CTA clears them.
bool Executor::reserve_scratch(size_t tiles) {
    if (tiles <= scratch_tiles_) return true;
    if (!check(cudaDeviceSynchronize(), "synchronise")) return false;
    cudaFree(d_scratch_); cudaFree(d_counters_);
    d_scratch_ = nullptr; d_counters_ = nullptr; scratch_tiles_ = 0;
    const size_t sb = tiles * 64u * kTileM * sizeof(float), cb = tiles * sizeof(uint32_t);
    if (!check(cudaMalloc(&d_scratch_, sb), "split-K scratch allocation") || !check(cudaMalloc(&d_counters_, cb), "split-K counter allocation"))
        return false;
    if (!check(cudaMemset(d_scratch_, 0, sb), "scratch clear") || !check(cudaMemset(d_counters_, 0, cb), "counter clear")) return false;
    scratch_tiles_ = tiles;
    drop_graph();
    return true;
}

void Executor::drop_graph() {
    if (graph_exec_) { cudaGraphExecDestroy(graph_exec_); graph_exec_ = nullptr; }
}

// Wave scheduler. Consecutive small waves that cannot observe each other (none reads or overwrites what another
// one writes) share one launch: their clusters are numbered consecutively in one grid. A decoder layer's q, k, v
// projections become one launch, gate and up another.
void Executor::build_groups() {
    groups_.clear();
    auto overlaps = [](uint64_t a0, uint64_t a1, uint64_t b0, uint64_t b1) { return a0 < b1 && b0 < a1; };
    bool allow = true;
    if (const char *e = std::getenv("K44B_GROUP")) allow = std::atoi(e) != 0;
    for (size_t i = 0; i < waves_.size(); ++i) {
        DeviceWave &w = waves_[i];
        bool joined = false;
        if (allow && w.groupable && !groups_.empty()) {
            LaunchGroup &g = groups_.back();
            const DeviceWave &first = waves_[g.waves[0]];
            bool ok = first.groupable && g.waves.size() < (size_t)kMaxGroupWaves && first.args.box_h == w.args.box_h;
            for (size_t k = 0; ok && k < g.waves.size(); ++k) {
                const DeviceWave &o = waves_[g.waves[k]];
                ok = !overlaps(w.read_lo, w.read_hi, o.write_lo, o.write_hi) && !overlaps(w.write_lo, w.write_hi, o.write_lo, o.write_hi) &&
                     !overlaps(w.write_lo, w.write_hi, o.read_lo, o.read_hi);
            }
            if (ok) {
                uint32_t tiles = 0;
                for (size_t k : g.waves) tiles += ((waves_[k].args.cout + kTileM - 1) / kTileM) * waves_[k].args.num_col_tiles64;
                tiles += ((w.args.cout + kTileM - 1) / kTileM) * w.args.num_col_tiles64;
                ok = tiles <= 2u * (uint32_t)num_sms_;
            }
            if (ok) { g.waves.push_back(i); joined = true; }
        }
        if (!joined) { groups_.push_back(LaunchGroup()); groups_.back().waves.push_back(i); }
    }
    for (auto &g : groups_) {
        if (!waves_[g.waves[0]].use_cluster) continue;
        uint32_t tiles = 0, min_ks = ~0u;
        for (size_t k : g.waves) {
            tiles += ((waves_[k].args.cout + kTileM - 1) / kTileM) * waves_[k].args.num_col_tiles64;
            min_ks = std::min(min_ks, waves_[k].args.num_kstages);
        }
        uint32_t S = g.waves.size() == 1 ? waves_[g.waves[0]].args.k_splits : 8u;
        if (g.waves.size() > 1)
            while (S > 1 && (S * tiles > 2u * (uint32_t)num_sms_ || S * 2u > min_ks)) S >>= 1;
        g.args = WaveGroupArgs();
        g.args.count = (uint32_t)g.waves.size();
        g.args.splits = S;
        uint32_t first = 0;
        for (size_t k = 0; k < g.waves.size(); ++k) {
            DeviceWave &w = waves_[g.waves[k]];
            w.args.k_splits = S;
            w.args.kstages_per_split = (w.args.num_kstages + S - 1) / S;
            g.args.w[k] = w.args;
            g.args.first_cluster[k] = first;
            first += ((w.args.cout + kTileM - 1) / kTileM) * w.args.num_col_tiles64;
        }
        g.args.total_clusters = first;
    }
    for (size_t gi = 0; gi < groups_.size(); ++gi) {
        const uint32_t sl = peer_slack_.size() == groups_.size() ? peer_slack_[gi] : 0u;
        groups_[gi].peer_slack = sl;
        for (uint32_t k = 0; k < groups_[gi].args.count; ++k) groups_[gi].args.w[k].peer_slack = sl;
    }
    groups_valid_ = true;
}

size_t Executor::num_launches() {
    if (!groups_valid_) build_groups();
    return groups_.size();
}

bool Executor::launch_hulls(uint64_t *out, size_t capacity) {
    if (!ready()) return fail("executor not initialised");
    if (!groups_valid_) build_groups();
    if (capacity < groups_.size()) return fail("launch_hulls: buffer too small");
    for (size_t gi = 0; gi < groups_.size(); ++gi) {
        uint64_t h[4] = {~0ull, 0, ~0ull, 0};
        for (size_t k : groups_[gi].waves) {
            const DeviceWave &w = waves_[k];
            if (w.read_lo < w.read_hi) { h[0] = std::min(h[0], w.read_lo); h[1] = std::max(h[1], w.read_hi); }
            if (w.write_lo < w.write_hi) { h[2] = std::min(h[2], w.write_lo); h[3] = std::max(h[3], w.write_hi); }
        }
        if (h[0] > h[1]) h[0] = h[1] = 0;
        if (h[2] > h[3]) h[2] = h[3] = 0;
        std::memcpy(out + gi * 4u, h, sizeof h);
    }
    return true;
}

bool Executor::set_peer_hulls(int world, const uint64_t *hulls, size_t launches) {
    if (!ready()) return fail("executor not initialised");
    if (!d_peers_) return fail("set_peer_hulls: the peers have not been set");
    if (!groups_valid_) build_groups();
    if (world != peer_world_) return fail("set_peer_hulls: world size differs from set_peers");
    if (launches != groups_.size()) return fail("set_peer_hulls: the table has " + std::to_string(launches) + " launches per rank, this plan has " + std::to_string(groups_.size()));
    peer_slack_.assign(launches, 0u);
    compute_peer_slack(hulls, world, launches, peer_slack_.data());
    groups_valid_ = false;       // rebuilt with the new values at the next execution
    drop_graph();
    return true;
}

bool Executor::launch_group(size_t gi, cudaStream_t stream) {
    LaunchGroup &g = groups_[gi];
    DeviceWave &w0 = waves_[g.waves[0]];
    if (g.waves.size() == 1 && !w0.use_cluster) return launch_one(w0, stream, g.peer_slack);
    ++launches_;
    return check(launch_wave_umma_cluster(g.args, w0.desc, w0.tmap, pdl_, num_sms_, stream), ("launch of wave group starting at '" + w0.name + "'").c_str());
}

bool Executor::launch_one(DeviceWave &w, cudaStream_t stream, uint32_t peer_slack) {
    cudaError_t e;
    w.args.peer_slack = peer_slack;
    if (w.is_aux) {
        launches_ += (w.aux.kind == AUX_ROPE_ATTN || w.aux.kind == AUX_DECODE_ATTN) ? 3u : (w.aux.kind == AUX_ARGMAX ? 2u : 1u);
        return check(launch_aux(w.aux, pdl_, stream), ("launch of '" + w.name + "'").c_str());
    }
    if (w.path == PATH_UMMA && w.use_cluster) {
        WaveGroupArgs g;
        g.count = 1; g.splits = w.args.k_splits;
        g.w[0] = w.args;
        g.total_clusters = ((w.args.cout + kTileM - 1) / kTileM) * w.args.num_col_tiles64;
        e = launch_wave_umma_cluster(g, w.desc, w.tmap, pdl_, num_sms_, stream);
    } else if (w.path == PATH_UMMA && w.use_shift) {
        e = w.desc.ws_chunk ? launch_wave_umma_shift_ws(w.args, w.desc, w.tmap, num_sms_, stream) : launch_wave_umma_shift(w.args, w.desc, w.tmap, num_sms_, stream);
    } else if (w.path == PATH_UMMA && w.desc.pair && !w.args.peers) {
        e = launch_wave_umma_pair(w.args, w.desc, w.tmap, w.wmap, num_sms_, stream);
    } else if (w.path == PATH_UMMA) {
        w.args.scratch = d_scratch_;
        w.args.counters = d_counters_;
        UmmaDesc dd = w.desc;
        if (dd.pair) { dd.pair = 0; dd.idesc = make_umma_desc(dd.n_tile).idesc; }     // sharded plans: the one-CTA kernel
        e = launch_wave_umma(w.args, dd, w.tmap, num_sms_, stream);
    } else if (w.path == PATH_MMA) {
        e = launch_wave_mma(w.args, make_umma_desc(64).wait_cycles, stream);
    } else {
        e = launch_wave_fma(w.args, stream);
    }
    ++launches_;
    return check(e, ("launch of wave '" + w.name + "'").c_str());
}

bool Executor::execute(cudaStream_t stream) {
    if (!ready()) return fail("executor not initialised");
    if (!groups_valid_) build_groups();
    for (size_t gi = 0; gi < groups_.size(); ++gi)
        if (!launch_group(gi, stream)) return false;
    return true;
}

// The wave list is a fixed sequence: capture it once into a CUDA graph and replay it with one launch call.
bool Executor::execute_graph(cudaStream_t stream) {
    if (!ready()) return fail("executor not initialised");
    if (!graph_exec_) {
        cudaStream_t cap = nullptr;
        if (!check(cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking), "capture stream")) return false;
        cudaGraph_t g = nullptr;
        bool ok = check(cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal), "begin capture");
        const uint64_t before = launches_;
        if (ok) {
            ok = execute(cap);
            const cudaError_t e = cudaStreamEndCapture(cap, &g);
            if (ok) ok = check(e, "end capture");
        }
        launches_ = before;                    // capturing is not launching
        if (ok) ok = check(cudaGraphInstantiate(&graph_exec_, g, 0), "graph instantiate");
        if (g) cudaGraphDestroy(g);
        cudaStreamDestroy(cap);
        if (!ok) { graph_exec_ = nullptr; return false; }
    }
    launches_ += groups_.size();
    return check(cudaGraphLaunch(graph_exec_, stream), "graph launch");
}

bool Executor::execute_wave(size_t i, cudaStream_t stream) {
    if (!ready()) return fail("executor not initialised");
    if (i >= waves_.size()) return fail("wave index out of range");
    if (!groups_valid_) build_groups();     // fixes the split count a wave uses inside its group
    return launch_one(waves_[i], stream);
}

// Host FP16 in / out without any conversion: the input rows are copied straight into the canvas and the
// output rows straight out of it (both in canvas layout, `pitch` elements per row). With pinned host
// buffers the copies are asynchronous on `stream`; the call returns after the output has arrived.
bool Executor::infer_f16(const uint16_t *h_in, uint16_t *h_out, float *gpu_ms, cudaStream_t stream) {
    if (!ready()) return fail("executor not initialised");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    const size_t in_b = (size_t)in_c_ * pitch_ * 2, out_b = (size_t)out_c_ * pitch_ * 2;
    if (h_in && in_b && !check(cudaMemcpyAsync(canvas_ + in_off_, h_in, in_b, cudaMemcpyHostToDevice, stream), "input upload")) return false;
    if (!check(cudaEventRecord(ev0_, stream), "event record")) return false;
    if (!execute(stream)) return false;
    if (!check(cudaEventRecord(ev1_, stream), "event record")) return false;
    if (h_out && out_b && !check(cudaMemcpyAsync(h_out, canvas_ + out_off_, out_b, cudaMemcpyDeviceToHost, stream), "output download")) return false;
    if (!check(cudaStreamSynchronize(stream), "wave execution")) return false;
    float t = 0.f;
    cudaEventElapsedTime(&t, ev0_, ev1_);
    if (gpu_ms) *gpu_ms = t;
    uint32_t st = 0;
    if (!check(cudaMemcpy(&st, d_status_, 4, cudaMemcpyDeviceToHost), "status read")) return false;
    if (st) { recover_after_abort(); return fail(std::string("kernel status: ") + status_string(st)); }
    return true;
}

// Pipelined host I/O: `begin` uploads an inference's input rows into a staging buffer on a copy stream of its own; `next`
// completes that inference — staging -> canvas (device copy), waves, output download, all on `stream` — and, before it
// waits, starts the upload of the following inference's input, which then runs under this inference's waves and download.
// The staging buffer costs input_c * pitch * 2 bytes of device memory and one device copy per inference; what it buys is
// that the host link never idles while the GPU computes.
bool Executor::infer_f16_begin(const uint16_t *h_in) {
    if (!ready()) return fail("executor not initialised");
    if (!h_in) return fail("infer_f16_begin: null input");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    const size_t in_b = (size_t)in_c_ * pitch_ * 2;
    if (!in_b) return fail("infer_f16_begin: the plan has no input rows");
    if (!copy_stream_) {
        if (!check(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking), "copy stream") ||
            !check(cudaEventCreateWithFlags(&ev_uploaded_, cudaEventDisableTiming), "event") ||
            !check(cudaEventCreateWithFlags(&ev_stage_free_, cudaEventDisableTiming), "event") ||
            !check(cudaMalloc(&d_stage_in_, in_b), "staging buffer allocation"))
            return false;
    }
    if (stage_pending_) return fail("infer_f16_begin: the staged input has not been consumed yet");
    if (!check(cudaStreamWaitEvent(copy_stream_, ev_stage_free_, 0), "stream wait") ||        // (an event never recorded counts as complete)
        !check(cudaMemcpyAsync(d_stage_in_, h_in, in_b, cudaMemcpyHostToDevice, copy_stream_), "input upload") ||
        !check(cudaEventRecord(ev_uploaded_, copy_stream_), "event record"))
        return false;
    stage_pending_ = true;
    return true;
}

bool Executor::infer_f16_next(const uint16_t *h_in_next, uint16_t *h_out, float *gpu_ms, cudaStream_t stream) {
    if (!ready()) return fail("executor not initialised");
    if (!stage_pending_) return fail("infer_f16_next: no staged input (call infer_f16_begin first)");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    const size_t in_b = (size_t)in_c_ * pitch_ * 2, out_b = (size_t)out_c_ * pitch_ * 2;
    if (!check(cudaStreamWaitEvent(stream, ev_uploaded_, 0), "stream wait") ||
        !check(cudaMemcpyAsync(canvas_ + in_off_, d_stage_in_, in_b, cudaMemcpyDeviceToDevice, stream), "staging copy") ||
        !check(cudaEventRecord(ev_stage_free_, stream), "event record"))
        return false;
    stage_pending_ = false;
    if (h_in_next && !infer_f16_begin(h_in_next)) return false;          // runs under the waves below
    if (!check(cudaEventRecord(ev0_, stream), "event record")) return false;
    if (!execute(stream)) return false;
    if (!check(cudaEventRecord(ev1_, stream), "event record")) return false;
    if (h_out && out_b && !check(cudaMemcpyAsync(h_out, canvas_ + out_off_, out_b, cudaMemcpyDeviceToHost, stream), "output download")) return false;
    if (!check(cudaStreamSynchronize(stream), "wave execution")) return false;
    float t = 0.f;
    cudaEventElapsedTime(&t, ev0_, ev1_);
    if (gpu_ms) *gpu_ms = t;
    uint32_t st = 0;
    if (!check(cudaMemcpy(&st, d_status_, 4, cudaMemcpyDeviceToHost), "status read")) return false;
    if (st) { recover_after_abort(); return fail(std::string("kernel status: ") + status_string(st)); }
    return true;
}

// After a kernel gave up (any status bit), CTAs that returned early never reached the split-K arrival counters, and
// the CTAs of a sharded launch may not all have been counted: partial sums, counters and the per-launch CTA count are
// put back to their between-launches state so that the next execution starts clean.
void Executor::recover_after_abort() {
    cudaMemset(d_status_, 0, 4);
    if (d_scratch_) cudaMemset(d_scratch_, 0, scratch_tiles_ * 64u * kTileM * sizeof(float));
    if (d_counters_) cudaMemset(d_counters_, 0, scratch_tiles_ * sizeof(uint32_t));
    if (d_sync_) cudaMemset(d_sync_ + kSyncDone, 0, sizeof(uint32_t));
    cudaDeviceSynchronize();
}

bool Executor::read_status(uint32_t *status) {
    if (!ready()) return fail("executor not initialised");
    uint32_t st = 0;
    if (!check(cudaSetDevice(device_), "cudaSetDevice") || !check(cudaDeviceSynchronize(), "synchronise") ||
        !check(cudaMemcpy(&st, d_status_, 4, cudaMemcpyDeviceToHost), "status read"))
        return false;
    if (status) *status = st;
    if (st) { recover_after_abort(); err = std::string("kernel status: ") + status_string(st); }
    return true;
}

// ---- neuron sharding over several GPUs ---------------------------------------------------------------------
void *Executor::sync_ptr() {
    if (!ready()) { fail("executor not initialised"); return nullptr; }
    if (!d_sync_) {
        if (!check(cudaSetDevice(device_), "cudaSetDevice") || !check(cudaMalloc(&d_sync_, kSyncWords * sizeof(uint32_t)), "sync block allocation") ||
            !check(cudaMemset(d_sync_, 0, kSyncWords * sizeof(uint32_t)), "sync block clear") || !check(cudaDeviceSynchronize(), "sync block clear"))
            return nullptr;
    }
    return d_sync_;
}

bool Executor::ipc_handles(void *canvas_handle64, void *sync_handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!sync_ptr()) return false;
    cudaIpcMemHandle_t hc, hs;
    if (!check(cudaIpcGetMemHandle(&hc, canvas_), "canvas IPC handle") || !check(cudaIpcGetMemHandle(&hs, d_sync_), "sync IPC handle")) return false;
    std::memcpy(canvas_handle64, &hc, 64);
    std::memcpy(sync_handle64, &hs, 64);
    return true;
}

bool Executor::set_peers_ipc(int rank, int world, const void *canvas_handles, const void *sync_handles) {
    if (world < 2 || world > kMaxPeers + 1 || rank < 0 || rank >= world) return fail("set_peers: bad rank / world size");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    std::vector<void *> cp((size_t)world, nullptr), sp((size_t)world, nullptr);
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        cudaIpcMemHandle_t hc, hs;
        std::memcpy(&hc, (const char *)canvas_handles + 64 * (size_t)r, 64);
        std::memcpy(&hs, (const char *)sync_handles + 64 * (size_t)r, 64);
        if (!check(cudaIpcOpenMemHandle(&cp[r], hc, cudaIpcMemLazyEnablePeerAccess), "open peer canvas")) return false;
        ipc_opened_.push_back(cp[r]);
        if (!check(cudaIpcOpenMemHandle(&sp[r], hs, cudaIpcMemLazyEnablePeerAccess), "open peer sync block")) return false;
        ipc_opened_.push_back(sp[r]);
    }
    return set_peers_raw(rank, world, cp.data(), sp.data());
}

bool Executor::set_peers_raw(int rank, int world, void *const *canvas_ptrs, void *const *sync_ptrs) {
    if (!ready()) return fail("executor not initialised");
    if (world < 2 || world > kMaxPeers + 1 || rank < 0 || rank >= world) return fail("set_peers: bad rank / world size");
    for (const auto &w : waves_)
        if ((w.path != PATH_UMMA && w.path != PATH_MMA) || w.use_shift || w.args.tile_off_x)
            return fail("set_peers: '" + w.name + "' does not run on a kernel that stores to peers (" +
                        (w.use_shift ? std::string("token-shifted runs") : w.is_aux ? std::string("element-wise command") : std::string("FP32-FMA kernel")) + ")");
    if (!sync_ptr()) return false;
    PeerArgs pa;
    pa.sync = d_sync_;
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        if (!canvas_ptrs[r] || !sync_ptrs[r]) return fail("set_peers: missing pointer for rank " + std::to_string(r));
        const uint32_t q = pa.n_peers++;
        pa.canvas[q] = (__half *)canvas_ptrs[r];
        // the word of rank `rank` in rank r's block: its position in r's peer list
        pa.arrive[q] = (uint32_t *)sync_ptrs[r] + (rank < r ? rank : rank - 1);
    }
    if (!d_peers_ && !check(cudaMalloc(&d_peers_, sizeof(PeerArgs)), "peer table allocation")) return false;
    if (!check(cudaMemcpy(d_peers_, &pa, sizeof(PeerArgs), cudaMemcpyHostToDevice), "peer table upload")) return false;
    std::vector<void *> peer_canvases;
    for (int r = 0; r < world; ++r)
        if (r != rank) peer_canvases.push_back(canvas_ptrs[r]);
    for (auto &w : waves_) {
        w.args.peers = d_peers_;
        if (w.d_out_maps && !upload_out_maps(w, peer_canvases.data(), (uint32_t)peer_canvases.size())) return false;
    }
    peer_rank_ = rank; peer_world_ = world;
    peer_canvas_.assign(canvas_ptrs, canvas_ptrs + world);
    peer_sync_.assign(sync_ptrs, sync_ptrs + world);
    peer_canvas_[rank] = nullptr; peer_sync_[rank] = nullptr;
    groups_valid_ = false;
    drop_graph();
    return true;
}

bool Executor::peer_latency(int peer_rank, bool initiator, uint32_t iters, uint32_t payload_bytes, float *ns, cudaStream_t stream) {
    if (!ready() || !d_peers_) return fail("peer_latency: the peers have not been set");
    if (peer_rank < 0 || peer_rank >= peer_world_ || peer_rank == peer_rank_ || !peer_sync_[peer_rank]) return fail("peer_latency: bad peer rank");
    if (iters == 0 || iters > 1000000u || payload_bytes % 16u || (uint64_t)payload_bytes > canvas_elems_ * 2u) return fail("peer_latency: bad iteration count or payload size");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    unsigned long long *d_out = reinterpret_cast<unsigned long long *>(d_sync_ + 12);       // words 12..15 of the own sync block
    const cudaError_t e = launch_peer_pingpong(d_sync_ + kSyncProbe, (uint32_t *)peer_sync_[peer_rank] + kSyncProbe, peer_canvas_[peer_rank], payload_bytes,
                                               initiator, iters, probe_base_, make_umma_desc(64).wait_cycles, d_out, stream);
    if (!check(e, "latency probe launch")) return false;
    ++launches_;
    probe_base_ += iters;
    unsigned long long h[2] = {0, 0};
    if (!check(cudaMemcpyAsync(h, d_out, sizeof h, cudaMemcpyDeviceToHost, stream), "latency probe result") || !check(cudaStreamSynchronize(stream), "latency probe")) return false;
    if (h[1] != iters) return fail("peer_latency: timed out waiting for the peer after " + std::to_string(h[1]) + " round trips");
    if (ns) *ns = (float)((double)h[0] / (double)iters);
    return true;
}

bool Executor::execute_timed(float *ms) {
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    if (!check(cudaEventRecord(ev0_, nullptr), "event record")) return false;
    if (!execute(nullptr)) return false;
    if (!check(cudaEventRecord(ev1_, nullptr), "event record") || !check(cudaEventSynchronize(ev1_), "wave execution")) return false;
    float t = 0.f;
    cudaEventElapsedTime(&t, ev0_, ev1_);
    if (ms) *ms = t;
    uint32_t st = 0;
    if (!read_status(&st)) return false;
    return st == 0;
}

// Host FP32 in / out, the contract of the reference's infer_f32 (wavec/k44_wave_executor.cu:599-618):
// input is dense [C][W] FP32, converted to FP16 RTE into the padded input rows; gpu_ms covers the waves
// only; at most out_elems values are copied back. The FP32<->FP16 layout conversion runs on the device.
bool Executor::infer_f32(const float *h_in, int in_elems, float *h_out, int out_elems, float *gpu_ms) {
    if (!ready()) return fail("executor not initialised");
    if (!check(cudaSetDevice(device_), "cudaSetDevice")) return false;
    const size_t in_n = is_2d_ ? (size_t)std::max(1u, in2d_.frames) * in_c_ * in2d_.H * in2d_.W : (size_t)in_c_ * io_width_;
    const size_t out_n = is_2d_ ? (size_t)std::max(1u, out2d_.frames) * out_c_ * out2d_.H * out2d_.W : (size_t)out_c_ * io_width_;
    if (in_elems < 0 || (size_t)in_elems < in_n) return fail("input has fewer elements than the plan's input tensor");
    if (!d_in_f32_ && !check(cudaMalloc(&d_in_f32_, std::max<size_t>(in_n, 1) * 4), "input staging")) return false;
    if (!d_out_f32_ && !check(cudaMalloc(&d_out_f32_, std::max<size_t>(out_n, 1) * 4), "output staging")) return false;
    if (!check(cudaMemcpyAsync(d_in_f32_, h_in, in_n * 4, cudaMemcpyHostToDevice, nullptr), "input upload")) return false;
    if (is_2d_) {
        if (!check(launch_f32_to_planes(d_in_f32_, canvas_ + in_off_, in_c_, in2d_.H, in2d_.W, in2d_.W_pad, in2d_.ch_stride, std::max(1u, in2d_.frames), in2d_.frame_stride ? in2d_.frame_stride : in2d_.ch_stride, nullptr), "input conversion")) return false;
    } else if (!check(launch_f32_to_canvas(d_in_f32_, canvas_ + in_off_, in_c_, io_width_, pitch_, nullptr), "input conversion")) return false;
    ++launches_;
    if (!check(cudaEventRecord(ev0_, nullptr), "event record")) return false;
    if (!execute(nullptr)) return false;
    if (!check(cudaEventRecord(ev1_, nullptr), "event record")) return false;
    if (is_2d_) {
        if (!check(launch_planes_to_f32(canvas_ + out_off_, d_out_f32_, out_c_, out2d_.H, out2d_.W, out2d_.W_pad, out2d_.ch_stride, std::max(1u, out2d_.frames), out2d_.frame_stride ? out2d_.frame_stride : out2d_.ch_stride, nullptr), "output conversion")) return false;
    } else if (!check(launch_canvas_to_f32(canvas_ + out_off_, d_out_f32_, out_c_, io_width_, pitch_, nullptr), "output conversion")) return false;
    ++launches_;
    const size_t copy_n = std::min((size_t)std::max(out_elems, 0), out_n);
    if (!check(cudaMemcpy(h_out, d_out_f32_, copy_n * 4, cudaMemcpyDeviceToHost), "output download")) return false;
    float t = 0.f;
    cudaEventElapsedTime(&t, ev0_, ev1_);
    if (gpu_ms) *gpu_ms = t;
    uint32_t st = 0;
    if (!read_status(&st)) return false;
    return st == 0;
}

bool Executor::weights_to_rowmajor(size_t wave, void *d_dst) {
    if (wave >= waves_.size()) return fail("wave index out of range");
    const auto &w = waves_[wave];
    return check(launch_tiled_to_rowmajor((const uint4 *)w.d_weights, (uint4 *)d_dst, w.args.cout, w.args.fan_in, nullptr), "weight unpack") &&
           check(cudaDeviceSynchronize(), "weight unpack");
}

}  // namespace k44b
