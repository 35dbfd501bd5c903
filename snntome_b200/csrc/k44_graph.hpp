// Graph -> wave plan for the part of the reference's front end that 1-D token models need: Input, dense
// linears (1x1 convolutions, optional residual), the zero-copy topology nodes Split / Slice / Concat, and
// the element-wise / attention nodes of a decoder layer (RMSNorm with optional folding of its scale into the
// consuming linears, SwiGLU product, rotary embedding + causal grouped-query attention). The 2-D part of the
// reference compiler (image layouts, pooling, deconvolution) is not built; those builder calls report failure
// and leave the graph unchanged.
//
// Rules reproduced (not code): batch>1 on a [C,1,1] input becomes the token axis
// (wavec/k44_wave_compiler.hpp:78-83); padding of rows / fan-in and group-size choice
// (wavec/k44_plan_types.hpp:157-186); canvas placement by liveness with best-fit reuse, 64-element
// granularity and a final round-up to 128 (wavec/k44_wave_compiler.hpp:388-593); gather-table and
// weight ordering of a 1x1 wave with zero-filled padding slots (:746-779); index rebasing when an
// offset reaches 0x70000000 (:1061-1072); summary JSON keys (:1345-1405); RMSNorm scale folding: when every
// consumer of a normalised tensor is a linear, column c of their weights is multiplied by gamma[c] and the
// normaliser runs without a scale (:233-301).
#pragma once
#include <set>

#include "k44_host.hpp"

namespace k44b {

struct GraphNode {
    enum Kind { INPUT, LINEAR, SPLIT, SLICE, CONCAT, RMSNORM, SWIGLU, ROPE_ATTN } kind = INPUT;
    std::string name;
    std::vector<std::string> ins, outs;
    std::string residual;
    std::vector<uint32_t> slice_sizes;
    uint32_t cin = 0, cout = 0, width = 1;
    int act = ACT_NONE;
    std::vector<uint16_t> w_f16;      // [cout][cin]
    std::vector<uint16_t> bias_f16;   // [cout]
    // RMSNorm: scale and epsilon; attention: head counts, rotary base
    std::vector<float> gamma;
    float eps = 1e-5f, rope_theta = 10000.0f;
    bool pre_folded = false, llama3_scaling = false, gamma_folded = false;
    uint32_t h_q = 0, h_kv = 0, head_dim = 0;
};

class WaveGraph {
  public:
    // options (wavec_create / wavec_set_*)
    uint32_t max_b_per_wave = 0, forced_group = 0, kv_cache_max_seq = 0, batch_size = 1;
    bool fold_rmsnorm_gamma = true, reuse_canvas = false;
    TargetPreset target;
    std::string output_tensor = "out0";

    std::vector<GraphNode> nodes;
    HostPlan plan;
    bool compiled = false;
    std::string summary_json = "{}";
    std::string error;

    bool add_input(const char *name, int c, int h, int w, int is_1d) {
        if (!name || c <= 0 || h <= 0 || w <= 0) return fail("add_input: bad arguments");
        const bool one_d = is_1d || (h == 1 && (w < 4 || w % 4 != 0));
        if (!one_d || h != 1) return fail("add_input: only 1-D token inputs [C,1,W] are supported by this library");
        GraphNode n;
        n.kind = GraphNode::INPUT; n.name = name; n.outs = {name}; n.cin = n.cout = (uint32_t)c; n.width = (uint32_t)w;
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }

    // Shared by the f32 / f16 / bf16 entry points; `w` is already FP16, row-major [cout][cin].
    bool add_linear(const char *name, const char *in, const char *out, int cin, int cout, int act,
                    std::vector<uint16_t> &&w, const float *bias_f32, const char *residual) {
        if (!name || !in || !out || cin <= 0 || cout <= 0) return fail("add_linear: bad arguments");
        if (act < 0 || act > ACT_GELU) return fail("add_linear: unknown activation");
        GraphNode n;
        n.kind = GraphNode::LINEAR; n.name = name; n.ins = {in}; n.outs = {out};
        n.cin = (uint32_t)cin; n.cout = (uint32_t)cout; n.act = act; n.w_f16 = std::move(w);
        n.bias_f16.assign((size_t)cout, 0);
        if (bias_f32) for (int i = 0; i < cout; ++i) n.bias_f16[i] = float_to_half(bias_f32[i]);
        if (residual && residual[0]) n.residual = residual;
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }

    bool add_topology(GraphNode::Kind kind, const char *name, std::vector<std::string> ins,
                      std::vector<std::string> outs, std::vector<uint32_t> sizes = {}) {
        if (!name || ins.empty() || outs.empty()) return fail("topology node: bad arguments");
        GraphNode n;
        n.kind = kind; n.name = name; n.ins = std::move(ins); n.outs = std::move(outs); n.slice_sizes = std::move(sizes);
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }

    bool add_rmsnorm(const char *name, const char *in, const char *out, int dim, float eps, const float *gamma, int pre_folded) {
        if (!name || !in || !out || dim <= 0) return fail("add_rmsnorm: bad arguments");
        GraphNode n;
        n.kind = GraphNode::RMSNORM; n.name = name; n.ins = {in}; n.outs = {out}; n.cin = n.cout = (uint32_t)dim; n.eps = eps;
        n.pre_folded = pre_folded != 0;
        if (gamma && !n.pre_folded) n.gamma.assign(gamma, gamma + dim);
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }

    bool add_swiglu(const char *name, const char *gate, const char *up, const char *out) {
        if (!name || !gate || !up || !out) return fail("add_swiglu: bad arguments");
        GraphNode n;
        n.kind = GraphNode::SWIGLU; n.name = name; n.ins = {gate, up}; n.outs = {out};
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }

    bool add_rope_attn(const char *name, const char *q, const char *k, const char *v, const char *out, int h_q, int h_kv, int head_dim,
                       float theta, int llama3) {
        if (!name || !q || !k || !v || !out || h_q <= 0 || h_kv <= 0 || h_q % h_kv) return fail("add_rope_gqa_attn: bad arguments");
        if (head_dim != 64 && head_dim != 128) return fail("add_rope_gqa_attn: head_dim must be 64 or 128");
        GraphNode n;
        n.kind = GraphNode::ROPE_ATTN; n.name = name; n.ins = {q, k, v}; n.outs = {out};
        n.h_q = (uint32_t)h_q; n.h_kv = (uint32_t)h_kv; n.head_dim = (uint32_t)head_dim; n.rope_theta = theta; n.llama3_scaling = llama3 != 0;
        n.cout = (uint32_t)(h_q * head_dim);
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }

    bool compile() {
        plan = HostPlan();
        compiled = false;
        if (nodes.empty() || nodes[0].kind != GraphNode::INPUT) return fail("compile: graph has no input");
        // ---- shapes -------------------------------------------------------------------------------
        uint32_t width = nodes[0].width;
        if (batch_size > 1 && width == 1) width = batch_size;      // batch becomes the token axis
        std::map<std::string, uint32_t> channels;                  // tensor -> channel count
        for (auto &n : nodes) {
            switch (n.kind) {
            case GraphNode::INPUT: channels[n.outs[0]] = n.cout; break;
            case GraphNode::LINEAR:
                if (!channels.count(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                if (channels[n.ins[0]] != n.cin) return fail("compile: " + n.name + " expects " + std::to_string(n.cin) + " input channels");
                if (n.w_f16.size() != (size_t)n.cin * n.cout) return fail("compile: " + n.name + " has no weights");
                if (!n.residual.empty() && (!channels.count(n.residual) || channels[n.residual] < n.cout))
                    return fail("compile: residual tensor of " + n.name + " is missing or too small");
                channels[n.outs[0]] = n.cout;
                break;
            case GraphNode::SPLIT:
                if (!channels.count(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                for (auto &o : n.outs) channels[o] = channels[n.ins[0]];
                break;
            case GraphNode::SLICE: {
                if (!channels.count(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                const uint32_t c = channels[n.ins[0]];
                uint32_t sum = 0;
                for (size_t k = 0; k < n.outs.size(); ++k) {
                    const uint32_t part = n.slice_sizes.empty() ? c / (uint32_t)n.outs.size() : n.slice_sizes[k];
                    channels[n.outs[k]] = part;
                    sum += part;
                }
                if (sum > c) return fail("compile: slice sizes exceed the tensor");
                break;
            }
            case GraphNode::CONCAT: {
                uint32_t sum = 0;
                for (auto &i : n.ins) {
                    if (!channels.count(i)) return fail("compile: unknown tensor " + i);
                    sum += channels[i];
                }
                channels[n.outs[0]] = sum;
                break;
            }
            case GraphNode::RMSNORM:
                if (!channels.count(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                if (channels[n.ins[0]] != n.cin) return fail("compile: " + n.name + " expects " + std::to_string(n.cin) + " channels");
                channels[n.outs[0]] = n.cout;
                break;
            case GraphNode::SWIGLU:
                if (!channels.count(n.ins[0]) || !channels.count(n.ins[1])) return fail("compile: unknown tensor at " + n.name);
                if (channels[n.ins[0]] != channels[n.ins[1]]) return fail("compile: " + n.name + ": gate and up differ in size");
                n.cin = n.cout = channels[n.ins[0]];
                channels[n.outs[0]] = n.cout;
                break;
            case GraphNode::ROPE_ATTN:
                for (auto &i : n.ins) if (!channels.count(i)) return fail("compile: unknown tensor " + i);
                if (channels[n.ins[0]] != n.h_q * n.head_dim || channels[n.ins[1]] != n.h_kv * n.head_dim || channels[n.ins[2]] != n.h_kv * n.head_dim)
                    return fail("compile: " + n.name + ": q / k / v channel counts do not match the head counts");
                channels[n.outs[0]] = n.cout;
                break;
            }
        }
        // ---- RMSNorm scale folding ------------------------------------------------------------------
        num_folded = 0;
        for (size_t s = 0; s < nodes.size(); ++s) {
            GraphNode &n = nodes[s];
            if (n.kind != GraphNode::RMSNORM || n.gamma.empty() || n.gamma_folded || !fold_rmsnorm_gamma) continue;
            bool ok = n.outs[0] != output_tensor;
            std::vector<size_t> users;
            for (size_t t = 0; t < nodes.size() && ok; ++t) {
                if (t == s) continue;
                const GraphNode &m = nodes[t];
                if (m.residual == n.outs[0]) ok = false;
                for (size_t k = 0; k < m.ins.size(); ++k)
                    if (m.ins[k] == n.outs[0]) { if (m.kind == GraphNode::LINEAR && k == 0) users.push_back(t); else ok = false; }
            }
            if (!ok || users.empty()) continue;
            for (size_t t : users) {
                GraphNode &m = nodes[t];
                for (uint32_t j = 0; j < m.cout; ++j)
                    for (uint32_t c = 0; c < m.cin; ++c) {
                        uint16_t &w = m.w_f16[(size_t)j * m.cin + c];
                        w = float_to_half(half_to_float(w) * n.gamma[c]);
                    }
            }
            n.gamma_folded = true;
        }
        for (auto &n : nodes) num_folded += (n.kind == GraphNode::RMSNORM && n.gamma_folded) ? 1 : 0;
        if (!channels.count(output_tensor)) {
            // default output = last produced tensor when "out0" was never defined
            output_tensor = nodes.back().outs[0];
        }
        plan.batch_size = std::max(1u, batch_size);
        plan.layout.init(width, 1);
        plan.target = target;
        plan.reuse_canvas = reuse_canvas;
        const uint32_t pitch = plan.layout.channel_stride;

        // ---- canvas placement ---------------------------------------------------------------------
        // allocation ids: one per Input / Linear node; topology nodes alias their sources
        std::map<std::string, std::set<int>> aliases;
        std::vector<int> node_aid(nodes.size(), -1);
        std::vector<uint32_t> aid_rows;
        for (size_t s = 0; s < nodes.size(); ++s) {
            auto &n = nodes[s];
            if (produces(n.kind)) {
                node_aid[s] = (int)aid_rows.size();
                aid_rows.push_back(n.kind == GraphNode::LINEAR ? pad_cout(n.cout) : n.cout);
                aliases[n.outs[0]] = {node_aid[s]};
            } else if (n.kind == GraphNode::CONCAT) {
                std::set<int> m;
                for (auto &i : n.ins) m.insert(aliases[i].begin(), aliases[i].end());
                aliases[n.outs[0]] = m;
            } else {
                for (auto &o : n.outs) aliases[o] = aliases[n.ins[0]];
            }
        }
        std::vector<size_t> last_use(aid_rows.size(), 0);
        last_use[0] = nodes.size();
        for (int a : aliases[output_tensor]) last_use[a] = nodes.size();
        for (size_t s = 0; s < nodes.size(); ++s) {
            for (auto &i : nodes[s].ins) for (int a : aliases[i]) last_use[a] = std::max(last_use[a], s);
            if (!nodes[s].residual.empty()) for (int a : aliases[nodes[s].residual]) last_use[a] = std::max(last_use[a], s);
        }
        struct Span { uint64_t at, len; };
        std::vector<Span> free_list;
        std::vector<uint64_t> aid_at(aid_rows.size(), 0), aid_len(aid_rows.size(), 0);
        std::set<int> live;
        uint64_t peak = 0;
        for (size_t s = 0; s < nodes.size(); ++s) {
            const int a = node_aid[s];
            if (a >= 0) {
                const uint64_t need = ((uint64_t)aid_rows[a] * pitch + 63u) & ~63ull;
                aid_len[a] = need;
                int best = -1;
                for (size_t k = 0; k < free_list.size(); ++k)
                    if (free_list[k].len >= need && (best < 0 || free_list[k].len < free_list[best].len)) best = (int)k;
                if (best >= 0) {
                    aid_at[a] = free_list[best].at;
                    if (free_list[best].len == need) free_list.erase(free_list.begin() + best);
                    else { free_list[best].at += need; free_list[best].len -= need; }
                } else if (!free_list.empty() && free_list.back().at + free_list.back().len == peak) {
                    aid_at[a] = free_list.back().at;         // grow the trailing hole
                    free_list.pop_back();
                    peak = aid_at[a] + need;
                } else {
                    aid_at[a] = peak;
                    peak += need;
                }
                live.insert(a);
            }
            bool retired = false;
            for (auto it = live.begin(); it != live.end();) {
                if (last_use[*it] <= s) { free_list.push_back({aid_at[*it], aid_len[*it]}); it = live.erase(it); retired = true; }
                else ++it;
            }
            if (retired && free_list.size() > 1) {
                std::sort(free_list.begin(), free_list.end(), [](const Span &x, const Span &y) { return x.at < y.at; });
                std::vector<Span> merged;
                for (auto &sp : free_list) {
                    if (!merged.empty() && merged.back().at + merged.back().len == sp.at) merged.back().len += sp.len;
                    else merged.push_back(sp);
                }
                free_list.swap(merged);
            }
        }
        uint64_t canvas = (peak + 63u) & ~63ull;
        canvas = (canvas + 127u) / 128u * 128u;
        if (canvas == 0) canvas = 128;
        if (canvas > 0xffffffffull) return fail("compile: canvas exceeds 2^32 FP16 elements");
        plan.canvas_elems = canvas;
        plan.input_off = aid_at[0];
        plan.input_c = nodes[0].cout; plan.input_h = 1; plan.input_w = width;

        // ---- command emission ---------------------------------------------------------------------
        std::map<std::string, std::vector<uint64_t>> rows_of;     // tensor -> canvas offset of every channel
        for (size_t s = 0; s < nodes.size(); ++s) {
            auto &n = nodes[s];
            if (produces(n.kind)) {
                std::vector<uint64_t> r(n.cout);
                for (uint32_t c = 0; c < n.cout; ++c) r[c] = aid_at[node_aid[s]] + (uint64_t)c * pitch;
                if (n.kind == GraphNode::LINEAR && !emit_linear(n, rows_of, aid_at[node_aid[s]])) return false;
                if (n.kind != GraphNode::LINEAR && n.kind != GraphNode::INPUT && !emit_aux(n, rows_of, aid_at[node_aid[s]])) return false;
                rows_of[n.outs[0]] = std::move(r);
            } else if (n.kind == GraphNode::SPLIT) {
                for (auto &o : n.outs) rows_of[o] = rows_of[n.ins[0]];
            } else if (n.kind == GraphNode::SLICE) {
                const auto &src = rows_of[n.ins[0]];
                size_t cur = 0;
                for (size_t k = 0; k < n.outs.size(); ++k) {
                    const size_t part = n.slice_sizes.empty() ? src.size() / n.outs.size() : n.slice_sizes[k];
                    rows_of[n.outs[k]] = std::vector<uint64_t>(src.begin() + cur, src.begin() + cur + part);
                    cur += part;
                }
            } else {
                std::vector<uint64_t> cat;
                for (auto &i : n.ins) cat.insert(cat.end(), rows_of[i].begin(), rows_of[i].end());
                rows_of[n.outs[0]] = std::move(cat);
            }
        }
        const auto &out_rows = rows_of[output_tensor];
        plan.output_off = out_rows.empty() ? 0 : out_rows[0];
        plan.output_c = plan.logical_output_c = channels[output_tensor];
        plan.output_h = 1; plan.output_w = width;
        compiled = true;
        build_summary();
        return true;
    }

  private:
    int num_folded = 0;
    bool fail(const std::string &m) { error = m; return false; }
    static bool produces(GraphNode::Kind k) {
        return k == GraphNode::INPUT || k == GraphNode::LINEAR || k == GraphNode::RMSNORM || k == GraphNode::SWIGLU || k == GraphNode::ROPE_ATTN;
    }
    // operands of the element-wise / attention kernels must be whole tensors: consecutive rows, `pitch` apart
    bool contiguous(const std::vector<uint64_t> &rows, uint32_t n) const {
        if (rows.size() < n) return false;
        for (uint32_t c = 1; c < n; ++c) if (rows[c] != rows[0] + (uint64_t)c * plan.layout.channel_stride) return false;
        return true;
    }

    bool emit_aux(GraphNode &n, std::map<std::string, std::vector<uint64_t>> &rows_of, uint64_t dst) {
        HostWave w;
        w.name = n.name; w.y_off = dst; w.cout = w.logical_cout = n.cout; w.cin = n.cin;
        w.h_out = 1; w.w_out = plan.layout.width;
        for (auto &i : n.ins)
            if (!contiguous(rows_of[i], (uint32_t)rows_of[i].size())) return fail("compile: " + n.name + " reads a tensor that is not stored as consecutive rows");
        w.src_off = rows_of[n.ins[0]][0];
        switch (n.kind) {
        case GraphNode::RMSNORM:
            w.kind = 1; w.eps = n.eps;
            if (!n.gamma.empty() && !n.gamma_folded) { w.bias.resize(n.cout); for (uint32_t c = 0; c < n.cout; ++c) w.bias[c] = float_to_half(n.gamma[c]); }
            break;
        case GraphNode::SWIGLU:
            w.kind = 2; w.src2_off = rows_of[n.ins[1]][0];
            break;
        case GraphNode::ROPE_ATTN:
            w.kind = 3; w.src2_off = rows_of[n.ins[1]][0]; w.src3_off = rows_of[n.ins[2]][0];
            w.h_q = n.h_q; w.h_kv = n.h_kv; w.head_dim = n.head_dim; w.rope_theta = n.rope_theta; w.llama3_scaling = n.llama3_scaling;
            w.seq_len = plan.layout.single_stride;          // one sequence per frame of the 1-D layout
            break;
        default: return fail("compile: unexpected node kind");
        }
        plan.waves.push_back(std::move(w));
        return true;
    }

    bool emit_linear(GraphNode &n, std::map<std::string, std::vector<uint64_t>> &rows_of, uint64_t dst) {
        const uint32_t pitch = plan.layout.channel_stride;
        const auto &in_rows = rows_of[n.ins[0]];
        HostWave w;
        w.name = n.name;
        w.cin = n.cin; w.logical_cout = n.cout; w.cout = pad_cout(n.cout);
        w.fan_in_raw = n.cin; w.fan_in = pad_fan_in(n.cin);
        w.group = choose_group_size(w.cout, std::max(1u, plan.layout.num_tiles), forced_group);
        w.act = n.act; w.has_bias = true;
        w.h_out = 1; w.w_out = plan.layout.width;
        w.y_off = dst; w.src_off = in_rows[0];
        if (!n.residual.empty()) {
            w.has_residual = true;
            w.res_off = rows_of[n.residual][0];
            // the epilogue reads `cout` padded rows of the residual: keep them inside the canvas
            const uint64_t end = w.res_off + (uint64_t)w.cout * pitch;
            if (end > plan.canvas_elems) plan.canvas_elems = (end + 127u) / 128u * 128u;
        }
        const uint32_t groups = w.cout / w.group;
        uint64_t lo = ~0ull, hi = 0;
        for (uint32_t c = 0; c < n.cin; ++c) { lo = std::min(lo, in_rows[c]); hi = std::max(hi, in_rows[c]); }
        if (hi >= 0x70000000ull) w.x_base_off = lo & ~63ull;
        w.idx.assign((size_t)groups * w.fan_in, 0u);
        for (uint32_t g = 0; g < groups; ++g)
            for (uint32_t c = 0; c < n.cin; ++c) w.idx[(size_t)g * w.fan_in + c] = (uint32_t)(in_rows[c] - w.x_base_off);
        w.bias.assign(w.cout, 0);
        std::copy(n.bias_f16.begin(), n.bias_f16.end(), w.bias.begin());
        std::vector<uint16_t> rm((size_t)w.cout * w.fan_in, 0);
        for (uint32_t j = 0; j < n.cout; ++j)
            std::memcpy(&rm[(size_t)j * w.fan_in], &n.w_f16[(size_t)j * n.cin], (size_t)n.cin * 2);
        w.w_wmma.resize(rm.size());
        rowmajor_to_wmma(rm.data(), w.w_wmma.data(), w.cout, w.fan_in);
        const double gf = 2.0 * (double)n.cin * (double)n.cout * (double)plan.layout.width / 1e9;
        w.gflops = gf;
        plan.single_frame_gflops += gf;
        plan.total_gflops += gf;
        plan.total_w_bytes += (uint64_t)w.cout * w.fan_in * 2;
        plan.total_idx_bytes += w.idx.size() * 4 + w.bias.size() * 2;
        plan.waves.push_back(std::move(w));
        return true;
    }

    void build_summary() {
        char buf[2048];
        std::snprintf(buf, sizeof buf,
                      "{\n  \"batch_size\": %u,\n  \"num_waves\": %zu,\n  \"num_cmds\": %zu,\n  \"canvas_elems\": %llu,\n"
                      "  \"canvas_bytes\": %llu,\n  \"kv_cache_elems\": 0,\n  \"total_w_bytes\": %llu,\n  \"total_idx_bytes\": %llu,\n"
                      "  \"single_frame_gflops\": %.6g,\n  \"total_gflops\": %.6g,\n  \"single_frame_gsyn\": %.6g,\n  \"total_gsyn\": %.6g,\n"
                      "  \"num_folded_rmsnorms\": %d,\n  \"num_eliminated_concats\": %d,\n  \"num_eliminated_splits\": %d,\n"
                      "  \"num_zero_copy_flattens\": 0,\n  \"input_shape\": [%u, %u, %u],\n  \"output_shape\": [%u, %u, %u],\n"
                      "  \"max_B_per_wave\": %u,\n  \"target_profile\": \"%s\",\n  \"target_num_cus\": %u,\n"
                      "  \"persistent_neurons\": %s,\n  \"reuse_canvas\": %s,\n  \"cmds\": [\n",
                      plan.batch_size, num_wave_cmds(), plan.waves.size(), (unsigned long long)plan.canvas_elems,
                      (unsigned long long)(plan.canvas_elems * 2ull), (unsigned long long)plan.total_w_bytes,
                      (unsigned long long)plan.total_idx_bytes, plan.single_frame_gflops, plan.total_gflops,
                      plan.single_frame_gflops * 0.5, plan.total_gflops * 0.5, num_folded, count(GraphNode::CONCAT),
                      count(GraphNode::SPLIT) + count(GraphNode::SLICE), plan.input_c, plan.input_h, plan.input_w,
                      plan.logical_output_c, plan.output_h, plan.output_w, max_b_per_wave, plan.target.name.c_str(),
                      plan.target.num_units, reuse_canvas ? "false" : "true", reuse_canvas ? "true" : "false");
        summary_json = buf;
        for (size_t i = 0; i < plan.waves.size(); ++i) {
            const HostWave &w = plan.waves[i];
            static const char *types[] = {"K44_WAVE", "RMSNORM", "SWIGLU", "ROPE_GQA_ATTN", "DECODE_GQA_ATTN"};
            std::snprintf(buf, sizeof buf,
                          "    {\"idx\": %zu, \"name\": \"%s\", \"type\": \"%s\", \"Cin\": %u, \"Cout\": %u, \"logical_Cout\": %u, "
                          "\"B\": %u, \"B_raw\": %u, \"S\": %u, \"act\": \"%s\", \"has_residual\": %s, \"has_self_read\": false, "
                          "\"subwave\": [0, 1], \"h_out\": %u, \"w_out\": %u, \"src_off\": %llu, \"y_off\": %llu, \"gflops\": %.6g}%s\n",
                          i, w.name.c_str(), types[w.kind >= 0 && w.kind <= 4 ? w.kind : 0], w.cin, w.cout, w.logical_cout, w.fan_in, w.fan_in_raw, w.group, act_name(w.act),
                          w.has_residual ? "true" : "false", w.h_out, w.w_out, (unsigned long long)w.src_off,
                          (unsigned long long)w.y_off, w.gflops, i + 1 < plan.waves.size() ? "," : "");
            summary_json += buf;
        }
        summary_json += "  ]\n}\n";
    }

    size_t num_wave_cmds() const {
        size_t c = 0;
        for (auto &w : plan.waves) c += w.kind == 0;
        return c;
    }

    int count(GraphNode::Kind k) const {
        int c = 0;
        for (auto &n : nodes) c += n.kind == k;
        return c;
    }
};

}  // namespace k44b
