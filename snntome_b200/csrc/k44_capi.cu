// extern "C" surface of libk44wavec.so: the reference-compatible wavec_* calls (include/k44wavec.h)
// and the native k44b_* additions (include/k44b.h).
#include <memory>
#include <mutex>

#include "../../include/k44b.h"
#include "../../include/k44wavec.h"
#include "k44_exec.hpp"
#include "k44_graph.hpp"
#include "k44_tcff.hpp"

using namespace k44b;

namespace {

thread_local std::string g_last_error;

int set_error(const std::string &m) {
    g_last_error = m;
    return -1;
}

struct NativePlan {
    Executor exec;
};

struct Handle {
    WaveGraph graph;
    std::unique_ptr<NativePlan> gpu;
    int device = 0;
    int force_path = -1;
};

Handle *H(void *p) { return static_cast<Handle *>(p); }
NativePlan *P(void *p) { return static_cast<NativePlan *>(p); }

bool ensure_compiled(Handle *h) {
    if (h->graph.compiled) return true;
    if (!h->graph.compile()) {
        set_error(h->graph.error);
        return false;
    }
    return true;
}

int add_linear_common(void *handle, const char *name, const char *in, const char *out, int din, int dout, int act,
                      std::vector<uint16_t> &&w, const float *bias, const char *res) {
    Handle *h = H(handle);
    if (!h) return set_error("null handle");
    return h->graph.add_linear(name, in, out, din, dout, act, std::move(w), bias, res) ? 0 : set_error(h->graph.error);
}

int unsupported(void *handle, const char *what) {
    if (!handle) return set_error("null handle");
    return set_error(std::string(what) + " is not part of the wave path implemented by this library");
}

bool desc_to_wave(const k44b_wave_desc *d, HostWave &w, std::string &err) {
    if (!d) { err = "null wave descriptor"; return false; }
    if (!d->weights) { err = "wave descriptor has no weights"; return false; }
    if (!d->idx && !d->run_rows) { err = "wave descriptor has neither an index table nor a run table"; return false; }
    if (d->cout == 0 || d->group == 0 || d->cout % d->group || d->fan_in == 0 || d->fan_in % 8u || d->cout % 16u) {
        err = "wave descriptor has inconsistent dimensions";
        return false;
    }
    w.name = d->name ? d->name : "wave";
    w.cout = d->cout; w.logical_cout = d->logical_cout ? d->logical_cout : d->cout; w.cin = d->cin;
    w.group = d->group; w.fan_in = d->fan_in; w.fan_in_raw = d->fan_in_raw ? d->fan_in_raw : d->fan_in;
    w.act = d->act; w.has_residual = d->has_residual != 0; w.has_bias = d->bias != nullptr;
    w.y_off = d->y_off; w.src_off = d->src_off; w.res_off = d->res_off; w.x_base_off = d->x_base_off;
    const size_t groups = d->cout / d->group;
    if (d->idx) w.idx.assign(d->idx, d->idx + groups * d->fan_in);
    if (d->run_rows) {
        if (d->run_len == 0 || d->fan_in % d->run_len) { err = "run length must divide the fan-in"; return false; }
        w.run_len = d->run_len;
        w.run_rows.assign(d->run_rows, d->run_rows + groups * (d->fan_in / d->run_len));
    }
    if (d->weights_on_device) {
        w.dev_weights_rowmajor = d->weights;
    } else {
        w.w_wmma.resize((size_t)d->cout * d->fan_in);
        rowmajor_to_wmma(d->weights, w.w_wmma.data(), d->cout, d->fan_in);
    }
    if (d->bias) w.bias.assign(d->bias, d->bias + d->cout);
    if (d->cout_map) w.cout_map.assign(d->cout_map, d->cout_map + d->cout);
    if (d->shifts) {
        const size_t n = d->run_rows ? groups * (d->fan_in / d->run_len) : groups * d->fan_in;
        w.shifts.assign(d->shifts, d->shifts + n);
    }
    w.frame_len = d->frame_len;
    if (d->num_tiles) {
        if (!d->tile_off_x || !d->tile_off_y || !d->plane_stride || !d->idx || d->weights_on_device) {
            err = "image wave: tile tables, plane stride, an index table and host weights are required";
            return false;
        }
        w.pitch2d = d->plane_stride;
        w.tile_mask = d->tile_mask != 0;
        w.tile_off_x.assign(d->tile_off_x, d->tile_off_x + d->num_tiles);
        w.tile_off_y.assign(d->tile_off_y, d->tile_off_y + d->num_tiles);
    }
    return true;
}

}  // namespace

extern "C" {

// ---------------------------------------------------------------------------------------------------
// reference-compatible surface
// ---------------------------------------------------------------------------------------------------
void *wavec_create(int max_B_per_wave, int default_S, int kv_cache_max_seq, int fold_rmsnorm_gamma) {
    Handle *h = new (std::nothrow) Handle();
    if (!h) return nullptr;
    h->graph.max_b_per_wave = (uint32_t)std::max(0, max_B_per_wave);
    h->graph.forced_group = (uint32_t)std::max(0, default_S);
    h->graph.kv_cache_max_seq = (uint32_t)std::max(0, kv_cache_max_seq);
    h->graph.fold_rmsnorm_gamma = fold_rmsnorm_gamma != 0;
    return h;
}

void wavec_destroy(void *handle) { delete H(handle); }

int wavec_gpu_release(void *handle) {
    if (!handle) return set_error("null handle");
    H(handle)->gpu.reset();
    return 0;
}

int wavec_add_input(void *handle, const char *name, int c, int h, int w, int is_1d) {
    if (!handle) return set_error("null handle");
    return H(handle)->graph.add_input(name, c, h, w, is_1d) ? 0 : set_error(H(handle)->graph.error);
}

int wavec_add_flatten(void *handle, const char *, const char *, const char *) { return unsupported(handle, "flatten"); }

int wavec_add_conv2d(void *handle, const char *name, const char *in, const char *out, int cin, int cout, int kh, int kw,
                     int stride, int pad, int act, const float *w_f32, const float *bias_f32, const char *res) {
    Handle *h = H(handle);
    if (!h) return set_error("null handle");
    if (!h->graph.is_2d) {       // token graphs: a 1x1 convolution is a linear
        if (kh != 1 || kw != 1 || stride != 1 || pad != 0) return set_error("add_conv2d: spatial convolutions need a 2-D image input");
        return wavec_add_linear_f32(handle, name, in, out, cin, cout, act, w_f32, bias_f32, res);
    }
    if (cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0) return set_error("add_conv2d: bad dimensions");
    std::vector<uint16_t> w((size_t)cin * cout * kh * kw, 0);
    if (w_f32) for (size_t i = 0; i < w.size(); ++i) w[i] = float_to_half(w_f32[i]);
    return h->graph.add_conv(name, in, out, cin, cout, kh, kw, stride, pad, act, std::move(w), bias_f32, res) ? 0 : set_error(h->graph.error);
}

int wavec_add_conv2d_f16(void *handle, const char *name, const char *in, const char *out, int cin, int cout, int kh, int kw,
                         int stride, int pad, int act, const uint16_t *w_f16, const float *bias_f32, const char *res) {
    Handle *h = H(handle);
    if (!h) return set_error("null handle");
    if (!h->graph.is_2d) {
        if (kh != 1 || kw != 1 || stride != 1 || pad != 0) return set_error("add_conv2d: spatial convolutions need a 2-D image input");
        return wavec_add_linear_f16(handle, name, in, out, cin, cout, act, w_f16, bias_f32, res);
    }
    if (cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0) return set_error("add_conv2d: bad dimensions");
    std::vector<uint16_t> w((size_t)cin * cout * kh * kw, 0);
    if (w_f16) std::memcpy(w.data(), w_f16, w.size() * 2);
    return h->graph.add_conv(name, in, out, cin, cout, kh, kw, stride, pad, act, std::move(w), bias_f32, res) ? 0 : set_error(h->graph.error);
}

int wavec_add_linear_f32(void *handle, const char *name, const char *in, const char *out, int din, int dout, int act,
                         const float *w_f32, const float *bias_f32, const char *res) {
    if (din <= 0 || dout <= 0) return set_error("add_linear: bad dimensions");
    std::vector<uint16_t> w((size_t)din * dout, 0);
    if (w_f32) for (size_t i = 0; i < w.size(); ++i) w[i] = float_to_half(w_f32[i]);
    return add_linear_common(handle, name, in, out, din, dout, act, std::move(w), bias_f32, res);
}

int wavec_add_linear_f16(void *handle, const char *name, const char *in, const char *out, int din, int dout, int act,
                         const uint16_t *w_f16, const float *bias_f32, const char *res) {
    if (din <= 0 || dout <= 0) return set_error("add_linear: bad dimensions");
    std::vector<uint16_t> w((size_t)din * dout, 0);
    if (w_f16) std::memcpy(w.data(), w_f16, w.size() * 2);
    return add_linear_common(handle, name, in, out, din, dout, act, std::move(w), bias_f32, res);
}

int wavec_add_linear_bf16(void *handle, const char *name, const char *in, const char *out, int din, int dout, int act,
                          const uint16_t *w_bf16, const float *bias_f32, const char *res) {
    if (din <= 0 || dout <= 0) return set_error("add_linear: bad dimensions");
    std::vector<uint16_t> w((size_t)din * dout, 0);
    if (w_bf16) for (size_t i = 0; i < w.size(); ++i) w[i] = float_to_half(bf16_to_float(w_bf16[i]));
    return add_linear_common(handle, name, in, out, din, dout, act, std::move(w), bias_f32, res);
}

int wavec_add_upconv2x2(void *handle, const char *name, const char *in, const char *out, int cin, int cout, const float *w_f32, const float *bias_f32) {
    if (!handle) return set_error("null handle");
    if (cin <= 0 || cout <= 0 || !w_f32) return set_error("add_upconv2x2: bad arguments");
    std::vector<uint16_t> w((size_t)cin * cout * 4u);
    for (size_t i = 0; i < w.size(); ++i) w[i] = float_to_half(w_f32[i]);
    return H(handle)->graph.add_upconv(name, in, out, cin, cout, std::move(w), bias_f32) ? 0 : set_error(H(handle)->graph.error);
}
int wavec_add_maxpool(void *handle, const char *name, const char *in, const char *out, int k, int stride, int pad) {
    if (!handle) return set_error("null handle");
    return H(handle)->graph.add_pool(name, in, out, k, stride, pad) ? 0 : set_error(H(handle)->graph.error);
}
int wavec_add_upsample2x(void *handle, const char *name, const char *in, const char *out) {
    if (!handle) return set_error("null handle");
    return H(handle)->graph.add_upsample(name, in, out) ? 0 : set_error(H(handle)->graph.error);
}
int wavec_add_rmsnorm(void *handle, const char *name, const char *in, const char *out, int dim, float eps, const float *gamma_f32, int pre_folded) {
    if (!handle) return set_error("null handle");
    return H(handle)->graph.add_rmsnorm(name, in, out, dim, eps, gamma_f32, pre_folded) ? 0 : set_error(H(handle)->graph.error);
}
int wavec_add_swiglu(void *handle, const char *name, const char *gate, const char *up, const char *out) {
    if (!handle) return set_error("null handle");
    return H(handle)->graph.add_swiglu(name, gate, up, out) ? 0 : set_error(H(handle)->graph.error);
}
int wavec_add_rope_gqa_attn(void *handle, const char *name, const char *q, const char *k, const char *v, const char *out, int h_q, int h_kv,
                            int head_dim, float rope_theta, int llama3_scaling) {
    if (!handle) return set_error("null handle");
    return H(handle)->graph.add_rope_attn(name, q, k, v, out, h_q, h_kv, head_dim, rope_theta, llama3_scaling) ? 0 : set_error(H(handle)->graph.error);
}

int wavec_add_split(void *handle, const char *name, const char *in, int n, const char **outs) {
    if (!handle || n <= 0 || !in || !outs) return set_error("add_split: bad arguments");
    std::vector<std::string> o(outs, outs + n);
    return H(handle)->graph.add_topology(GraphNode::SPLIT, name, {in}, o) ? 0 : set_error(H(handle)->graph.error);
}

int wavec_add_slice(void *handle, const char *name, const char *in, int n, const char **outs, const int *sizes) {
    if (!handle || n <= 0 || !in || !outs) return set_error("add_slice: bad arguments");
    std::vector<std::string> o(outs, outs + n);
    std::vector<uint32_t> sz;
    if (sizes) for (int i = 0; i < n; ++i) sz.push_back((uint32_t)std::max(0, sizes[i]));
    return H(handle)->graph.add_topology(GraphNode::SLICE, name, {in}, o, sz) ? 0 : set_error(H(handle)->graph.error);
}

int wavec_add_concat(void *handle, const char *name, int n, const char **ins, const char *out) {
    if (!handle || n <= 0 || !ins || !out) return set_error("add_concat: bad arguments");
    std::vector<std::string> i(ins, ins + n);
    return H(handle)->graph.add_topology(GraphNode::CONCAT, name, i, {out}) ? 0 : set_error(H(handle)->graph.error);
}

int wavec_set_output(void *handle, const char *out) {
    if (!handle || !out) return set_error("set_output: bad arguments");
    H(handle)->graph.output_tensor = out;
    H(handle)->graph.compiled = false;
    return 0;
}

int wavec_set_reuse_canvas(void *handle, int on) {
    if (!handle) return set_error("null handle");
    H(handle)->graph.reuse_canvas = on != 0;
    H(handle)->graph.compiled = false;
    return 0;
}

int wavec_set_batch_size(void *handle, int batch) {
    if (!handle) return set_error("null handle");
    H(handle)->graph.batch_size = (uint32_t)std::max(1, batch);
    H(handle)->graph.compiled = false;
    return 0;
}

int wavec_set_target_preset(void *handle, const char *preset) {
    if (!handle) return set_error("null handle");
    H(handle)->graph.target = preset_from_name(preset);
    H(handle)->graph.compiled = false;
    return 0;
}

int wavec_compile(void *handle) {
    if (!handle) return set_error("null handle");
    return H(handle)->graph.compile() ? 0 : set_error(H(handle)->graph.error);
}

const char *wavec_get_summary_json(void *handle) {
    if (!handle || !ensure_compiled(H(handle))) return "{}";
    return H(handle)->graph.summary_json.c_str();
}

int wavec_save_tcff_ex(void *handle, const char *path, const char *prefix, int /*include_canvas*/, int include_geometry) {
    if (!handle || !path) return set_error("save_tcff: bad arguments");
    if (!ensure_compiled(H(handle))) return -1;
    std::string err;
    return tcff_save(H(handle)->graph.plan, path, prefix, include_geometry != 0, err) ? 0 : set_error(err);
}

int wavec_save_tcff(void *handle, const char *path, const char *prefix) { return wavec_save_tcff_ex(handle, path, prefix, 1, 1); }

int wavec_load_tcff_weights(void *handle, const char *path) {
    if (!handle || !path) return set_error("load_tcff_weights: bad arguments");
    if (!ensure_compiled(H(handle))) return -1;
    std::string err;
    return tcff_load_into(H(handle)->graph.plan, path, err) ? 0 : set_error(err);
}

int wavec_gpu_init_plan(void *handle) {
    Handle *h = H(handle);
    if (!h) return set_error("null handle");
    if (!ensure_compiled(h)) return -1;
    std::unique_ptr<NativePlan> p(new NativePlan());
    if (!p->exec.init(h->graph.plan, h->device, h->force_path)) return set_error(p->exec.err);
    h->gpu = std::move(p);
    return 0;
}

int wavec_gpu_infer_f32(void *handle, const float *h_in, int in_elems, float *h_out, int out_elems, float *out_gpu_ms) {
    if (!handle || !h_in || !h_out) return set_error("gpu_infer_f32: bad arguments");
    Handle *h = H(handle);
    if (!h->gpu) return set_error("gpu_infer_f32: wavec_gpu_init_plan has not been called");
    return h->gpu->exec.infer_f32(h_in, in_elems, h_out, out_elems, out_gpu_ms) ? 0 : set_error(h->gpu->exec.err);
}

// ---------------------------------------------------------------------------------------------------
// native surface
// ---------------------------------------------------------------------------------------------------
void *k44b_plan_create(int device, uint64_t canvas_elems, uint32_t pitch, uint32_t columns, int force_path) {
    std::unique_ptr<NativePlan> p(new NativePlan());
    if (!p->exec.begin(device, canvas_elems, pitch, columns, force_path)) {
        set_error(p->exec.err);
        return nullptr;
    }
    return p.release();
}

int k44b_plan_add_wave(void *plan, const k44b_wave_desc *wave) {
    if (!plan) return set_error("null plan");
    HostWave w;
    std::string err;
    if (!desc_to_wave(wave, w, err)) return set_error(err);
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_add_rmsnorm(void *plan, const char *name, uint64_t src_off, uint64_t dst_off, uint32_t dim, float eps, const uint16_t *gamma_f16) {
    if (!plan || !dim) return set_error("plan_add_rmsnorm: bad arguments");
    HostWave w;
    w.kind = AUX_RMSNORM; w.name = name ? name : "rmsnorm"; w.cout = dim; w.src_off = src_off; w.y_off = dst_off; w.eps = eps;
    if (gamma_f16) w.bias.assign(gamma_f16, gamma_f16 + dim);
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_add_swiglu(void *plan, const char *name, uint64_t gate_off, uint64_t up_off, uint64_t dst_off, uint32_t rows) {
    if (!plan || !rows) return set_error("plan_add_swiglu: bad arguments");
    HostWave w;
    w.kind = AUX_SWIGLU; w.name = name ? name : "swiglu"; w.cout = rows; w.src_off = gate_off; w.src2_off = up_off; w.y_off = dst_off;
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_add_rope_attn(void *plan, const char *name, uint64_t q_off, uint64_t k_off, uint64_t v_off, uint64_t out_off, uint32_t h_q,
                            uint32_t h_kv, uint32_t head_dim, float rope_theta, int llama3_scaling, uint32_t seq_len) {
    if (!plan) return set_error("plan_add_rope_attn: bad arguments");
    HostWave w;
    w.kind = AUX_ROPE_ATTN; w.name = name ? name : "rope_attn"; w.cout = h_q * head_dim;
    w.src_off = q_off; w.src2_off = k_off; w.src3_off = v_off; w.y_off = out_off;
    w.h_q = h_q; w.h_kv = h_kv; w.head_dim = head_dim; w.rope_theta = rope_theta; w.llama3_scaling = llama3_scaling != 0; w.seq_len = seq_len;
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_add_decode_attn(void *plan, const char *name, uint64_t q_off, uint64_t k_off, uint64_t v_off, uint64_t out_off,
                              uint64_t kcache_off, uint64_t vcache_off, uint32_t h_q, uint32_t h_kv, uint32_t head_dim, uint32_t max_seq,
                              float rope_theta, int llama3_scaling) {
    if (!plan) return set_error("plan_add_decode_attn: bad arguments");
    HostWave w;
    w.kind = AUX_DECODE_ATTN; w.name = name ? name : "decode_attn"; w.cout = h_q * head_dim;
    w.src_off = q_off; w.src2_off = k_off; w.src3_off = v_off; w.y_off = out_off; w.kcache_off = kcache_off; w.vcache_off = vcache_off;
    w.h_q = h_q; w.h_kv = h_kv; w.head_dim = head_dim; w.max_seq = max_seq; w.rope_theta = rope_theta; w.llama3_scaling = llama3_scaling != 0;
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_add_embedding(void *plan, const char *name, const void *d_table_f16, uint32_t vocab, uint32_t dim, uint64_t dst_off) {
    if (!plan || !d_table_f16 || !vocab || !dim) return set_error("plan_add_embedding: bad arguments");
    HostWave w;
    w.kind = AUX_EMBED; w.name = name ? name : "embedding"; w.cout = dim; w.y_off = dst_off; w.dev_table = d_table_f16; w.vocab = vocab;
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_add_argmax(void *plan, const char *name, uint64_t src_off, uint32_t rows, int advance, uint32_t max_seq) {
    if (!plan || !rows) return set_error("plan_add_argmax: bad arguments");
    HostWave w;
    w.kind = AUX_ARGMAX; w.name = name ? name : "argmax"; w.cout = rows; w.src_off = src_off; w.advance = advance != 0; w.max_seq = max_seq;
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_set_tokens(void *plan, const int32_t *h_tokens, uint32_t n, void *stream) {
    if (!plan || !h_tokens) return set_error("plan_set_tokens: bad arguments");
    Executor &e = P(plan)->exec;
    int *d = e.tokens_ptr();
    if (!d) return set_error(e.err);
    if (n > e.pitch()) return set_error("plan_set_tokens: more tokens than columns");
    const cudaError_t r = cudaMemcpyAsync(d, h_tokens, (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, (cudaStream_t)stream);
    return r == cudaSuccess ? 0 : set_error(std::string("plan_set_tokens: ") + cudaGetErrorString(r));
}

int k44b_plan_get_next_tokens(void *plan, int32_t *h_tokens, uint32_t n, void *stream) {
    if (!plan || !h_tokens) return set_error("plan_get_next_tokens: bad arguments");
    Executor &e = P(plan)->exec;
    int *d = e.next_tokens_ptr();
    if (!d) return set_error(e.err);
    if (n > e.pitch()) return set_error("plan_get_next_tokens: more tokens than columns");
    cudaError_t r = cudaMemcpyAsync(h_tokens, d, (size_t)n * sizeof(int32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (r == cudaSuccess) r = cudaStreamSynchronize((cudaStream_t)stream);
    return r == cudaSuccess ? 0 : set_error(std::string("plan_get_next_tokens: ") + cudaGetErrorString(r));
}

int k44b_plan_add_image_op(void *plan, int op, const char *name, uint64_t src_off, uint64_t dst_off, uint32_t planes,
                           const k44b_plane_geom *in, const k44b_plane_geom *out) {
    if (!plan || !out || op < AUX_MAXPOOL2 || op > AUX_HALO_CLEAR || (op != AUX_HALO_CLEAR && !in)) return set_error("plan_add_image_op: bad arguments");
    HostWave w;
    w.kind = op; w.name = name ? name : "image_op"; w.src_off = src_off; w.y_off = dst_off; w.cout = w.logical_cout = planes;
    auto conv = [](const k44b_plane_geom *g) { HostWave::Geom2D r; r.H = g->h; r.W = g->w; r.W_pad = g->w_pad; r.ch_stride = g->plane_stride; return r; };
    w.out2d = conv(out);
    w.in2d = in ? conv(in) : w.out2d;
    return P(plan)->exec.add_wave(w) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_set_decode_pos(void *plan, int pos, void *stream) {
    if (!plan || pos < 0) return set_error("plan_set_decode_pos: bad arguments");
    int *d = P(plan)->exec.decode_pos_ptr();
    if (!d) return set_error(P(plan)->exec.err);
    // a 4-byte asynchronous copy from pageable memory is staged by the runtime before the call returns
    const cudaError_t e = cudaMemcpyAsync(d, &pos, sizeof(int), cudaMemcpyHostToDevice, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : set_error(std::string("plan_set_decode_pos: ") + cudaGetErrorString(e));
}

int k44b_plan_set_io(void *plan, uint64_t input_off, uint32_t input_c, uint64_t output_off, uint32_t output_c, uint32_t width) {
    if (!plan) return set_error("null plan");
    Executor &e = P(plan)->exec;
    if (input_off + (uint64_t)input_c * e.pitch() > e.canvas_elems() || output_off + (uint64_t)output_c * e.pitch() > e.canvas_elems() ||
        width > e.pitch())
        return set_error("input / output region leaves the canvas");
    e.set_io(input_off, input_c, output_off, output_c, width);
    return 0;
}

void *k44b_plan_from_tcff(const char *path, uint32_t pitch_hint, int device, int force_path) {
    if (!path) { set_error("null path"); return nullptr; }
    HostPlan hp;
    std::string err;
    if (!tcff_to_plan(path, pitch_hint, hp, err)) { set_error(err); return nullptr; }
    std::unique_ptr<NativePlan> p(new NativePlan());
    if (!p->exec.init(hp, device, force_path)) { set_error(p->exec.err); return nullptr; }
    return p.release();
}

void k44b_plan_destroy(void *plan) { delete P(plan); }

void *k44b_canvas_ptr(void *plan) { return plan ? (void *)P(plan)->exec.canvas() : nullptr; }
uint64_t k44b_canvas_elems(void *plan) { return plan ? P(plan)->exec.canvas_elems() : 0; }
int k44b_num_waves(void *plan) { return plan ? (int)P(plan)->exec.num_waves() : -1; }

int k44b_wave_info(void *plan, int wave, k44b_wave_info_t *out) {
    if (!plan || !out || wave < 0 || (size_t)wave >= P(plan)->exec.num_waves()) return set_error("wave_info: bad arguments");
    const DeviceWave &w = P(plan)->exec.wave((size_t)wave);
    out->cout = w.args.cout; out->group = w.args.group; out->fan_in = w.args.fan_in;
    out->box_rows = w.args.gather_mode == GATHER_BOX ? w.args.box_h : 0;
    out->path = w.path; out->n_tile = w.path == PATH_UMMA ? w.desc.n_tile : 64;
    out->k_splits = w.path == PATH_UMMA ? w.args.k_splits : 1;
    out->synapses = w.synapses; out->weight_bytes = w.weight_bytes;
    out->m_blocks = (w.path == PATH_UMMA && !w.use_cluster && !w.use_shift) ? (w.desc.pair ? 2u : w.desc.m_blocks) : 1u;
    out->cta_pairs = (w.path == PATH_UMMA && !w.use_cluster && !w.use_shift) ? w.desc.pair : 0u;
    out->weights_in_tmem = (w.path == PATH_UMMA && w.use_shift) ? w.desc.ws_chunk : 0u;
    out->reserved0 = 0u;
    return 0;
}

int k44b_execute(void *plan, void *stream) {
    if (!plan) return set_error("null plan");
    return P(plan)->exec.execute((cudaStream_t)stream) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_execute_graph(void *plan, void *stream) {
    if (!plan) return set_error("null plan");
    return P(plan)->exec.execute_graph((cudaStream_t)stream) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_execute_wave(void *plan, int wave, void *stream) {
    if (!plan || wave < 0) return set_error("execute_wave: bad arguments");
    return P(plan)->exec.execute_wave((size_t)wave, (cudaStream_t)stream) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_infer_f16_begin(void *plan, const uint16_t *h_in) {
    if (!plan) return set_error("null plan");
    return P(plan)->exec.infer_f16_begin(h_in) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_infer_f16_next(void *plan, const uint16_t *h_in_next, uint16_t *h_out, float *out_gpu_ms, void *stream) {
    if (!plan) return set_error("null plan");
    return P(plan)->exec.infer_f16_next(h_in_next, h_out, out_gpu_ms, (cudaStream_t)stream) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_infer_f16(void *plan, const uint16_t *h_in, uint16_t *h_out, float *out_gpu_ms, void *stream) {
    if (!plan) return set_error("null plan");
    return P(plan)->exec.infer_f16(h_in, h_out, out_gpu_ms, (cudaStream_t)stream) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_status(void *plan, uint32_t *status) {
    if (!plan) return set_error("null plan");
    uint32_t st = 0;
    if (!P(plan)->exec.read_status(&st)) return set_error(P(plan)->exec.err);
    if (status) *status = st;
    return st == 0 ? 0 : set_error(P(plan)->exec.err);
}

int k44b_infer_f32(void *plan, const float *h_in, int in_elems, float *h_out, int out_elems, float *out_gpu_ms) {
    if (!plan || !h_in || !h_out) return set_error("infer_f32: bad arguments");
    return P(plan)->exec.infer_f32(h_in, in_elems, h_out, out_elems, out_gpu_ms) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_ipc_handles(void *plan, void *canvas_handle64, void *sync_handle64) {
    if (!plan || !canvas_handle64 || !sync_handle64) return set_error("plan_ipc_handles: bad arguments");
    return P(plan)->exec.ipc_handles(canvas_handle64, sync_handle64) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_set_peers_ipc(void *plan, int rank, int world, const void *canvas_handles, const void *sync_handles) {
    if (!plan || !canvas_handles || !sync_handles) return set_error("plan_set_peers_ipc: bad arguments");
    return P(plan)->exec.set_peers_ipc(rank, world, canvas_handles, sync_handles) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_set_peers_raw(void *plan, int rank, int world, void *const *canvas_ptrs, void *const *sync_ptrs) {
    if (!plan || !canvas_ptrs || !sync_ptrs) return set_error("plan_set_peers_raw: bad arguments");
    return P(plan)->exec.set_peers_raw(rank, world, canvas_ptrs, sync_ptrs) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_num_launches(void *plan) {
    if (!plan) return set_error("plan_num_launches: bad arguments");
    return (int)P(plan)->exec.num_launches();
}

int k44b_plan_launch_hulls(void *plan, uint64_t *out, uint64_t capacity) {
    if (!plan || !out) return set_error("plan_launch_hulls: bad arguments");
    return P(plan)->exec.launch_hulls(out, (size_t)capacity) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_plan_set_peer_hulls(void *plan, int world, const uint64_t *hulls, uint64_t launches) {
    if (!plan || !hulls) return set_error("plan_set_peer_hulls: bad arguments");
    return P(plan)->exec.set_peer_hulls(world, hulls, (size_t)launches) ? 0 : set_error(P(plan)->exec.err);
}

void k44b_compute_peer_slack(const uint64_t *hulls, int world, uint64_t launches, uint32_t *out_slack) {
    if (hulls && out_slack && world > 0) k44b::compute_peer_slack(hulls, world, (size_t)launches, out_slack);
}

int k44b_plan_peer_latency(void *plan, int peer_rank, int initiator, uint32_t iters, uint32_t payload_bytes, float *out_ns_per_round_trip, void *stream) {
    if (!plan) return set_error("plan_peer_latency: bad arguments");
    return P(plan)->exec.peer_latency(peer_rank, initiator != 0, iters, payload_bytes, out_ns_per_round_trip, (cudaStream_t)stream) ? 0 : set_error(P(plan)->exec.err);
}

void *k44b_plan_sync_ptr(void *plan) {
    if (!plan) { set_error("plan_sync_ptr: bad arguments"); return nullptr; }
    void *p = P(plan)->exec.sync_ptr();
    if (!p) set_error(P(plan)->exec.err);
    return p;
}

uint64_t k44b_launch_count(void *plan) { return plan ? P(plan)->exec.launches() : 0; }

int k44b_wave_weights_rowmajor(void *plan, int wave, void *d_dst) {
    if (!plan || !d_dst || wave < 0) return set_error("wave_weights_rowmajor: bad arguments");
    return P(plan)->exec.weights_to_rowmajor((size_t)wave, d_dst) ? 0 : set_error(P(plan)->exec.err);
}

int k44b_set_device(void *handle, int device) {
    if (!handle || device < 0) return set_error("set_device: bad arguments");
    H(handle)->device = device;
    return 0;
}

int k44b_set_force_path(void *handle, int force_path) {
    if (!handle) return set_error("null handle");
    H(handle)->force_path = force_path;
    return 0;
}

void *k44b_handle_plan(void *handle) { return handle ? (void *)H(handle)->gpu.get() : nullptr; }

const char *k44b_last_error(void) { return g_last_error.c_str(); }
const char *k44b_version(void) { return "k44b 0.1 (sm_100a)"; }

int k44b_fill_normal_f16(void *d_dst, uint64_t n, uint64_t seed, float scale, void *stream) {
    if (!d_dst) return set_error("fill_normal_f16: null pointer");
    const cudaError_t e = launch_fill_normal_f16((__half *)d_dst, n, seed, scale, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : set_error(std::string("fill_normal_f16: ") + cudaGetErrorString(e));
}

uint64_t k44b_fnv1a64(const uint8_t *data, uint64_t len) { return fnv1a64(data, (size_t)len); }

void k44b_f32_to_f16(const float *src, uint16_t *dst, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) dst[i] = float_to_half(src[i]);
}

void k44b_rowmajor_to_wmma(const uint16_t *src, uint16_t *dst, uint32_t cout, uint32_t fan_in) { rowmajor_to_wmma(src, dst, cout, fan_in); }
void k44b_wmma_to_rowmajor(const uint16_t *src, uint16_t *dst, uint32_t cout, uint32_t fan_in) { wmma_to_rowmajor(src, dst, cout, fan_in); }

int k44b_analyze_gather(const k44b_wave_desc *wave, uint32_t pitch, uint64_t canvas_elems, uint32_t *out_box_rows, uint64_t capacity,
                        uint64_t *out_count) {
    if (!wave || pitch == 0) return set_error("analyze_gather: bad arguments");
    HostWave w;
    w.cout = wave->cout; w.group = wave->group; w.fan_in = wave->fan_in;
    w.fan_in_raw = wave->fan_in_raw ? wave->fan_in_raw : wave->fan_in;
    w.x_base_off = wave->x_base_off;
    if (w.cout == 0 || w.group == 0 || w.cout % w.group || w.fan_in == 0) return set_error("analyze_gather: inconsistent dimensions");
    const size_t groups = w.cout / w.group;
    if (wave->idx) w.idx.assign(wave->idx, wave->idx + groups * w.fan_in);
    else if (wave->run_rows && wave->run_len && w.fan_in % wave->run_len == 0) {
        w.run_len = wave->run_len;
        w.run_rows.assign(wave->run_rows, wave->run_rows + groups * (w.fan_in / wave->run_len));
    } else return set_error("analyze_gather: no gather table");
    const GatherPlan gp = analyze_gather(w, pitch, canvas_elems);
    if (out_count) *out_count = gp.box_rows.size();
    if (!gp.box_ok || gp.small_group) { g_last_error = gp.why_not; return 0; }     // not usable by the tcgen05 kernels
    if (out_box_rows) std::memcpy(out_box_rows, gp.box_rows.data(), std::min<uint64_t>(capacity, gp.box_rows.size()) * 4);
    return (int)gp.box_h;
}

}  // extern "C"
