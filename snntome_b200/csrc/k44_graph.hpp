// Graph -> wave plan for the part of the reference's front end that 1-D token models need: Input, dense
// linears (1x1 convolutions, optional residual), the zero-copy topology nodes Split / Slice / Concat, and
// the element-wise / attention nodes of a decoder layer (RMSNorm with optional folding of its scale into the
// consuming linears, SwiGLU product, rotary embedding + causal grouped-query attention) — and for 2-D image models:
// convolutions (1x1 / 3x3, stride 1 or 2) as waves over haloed planes whose gather offsets are the filter taps, 2x2
// transposed convolutions (a wave that produces the four output phases plus a scatter), max-pooling 2x2 / 5x5, nearest
// upsampling, with the same zero-copy topology nodes (compile_2d below; wavec/k44_wave_compiler.hpp:692-807 for the tap
// rule, wavec/k44_plan_types.hpp:517-600 for the plane layouts). One image per inference (batch 1).
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
    enum Kind { INPUT, LINEAR, SPLIT, SLICE, CONCAT, RMSNORM, SWIGLU, ROPE_ATTN, MAXPOOL, UPSAMPLE, UPCONV } kind = INPUT;
    uint32_t kh = 1, kw = 1, stride = 1, pad = 0, height = 1;       // convolution / pooling window; input height
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
    bool is_2d = false;              // the input is an image [C][H][W] with H > 1: every tensor lives in haloed planes
    std::string summary_json = "{}";
    std::string error;

    bool add_input(const char *name, int c, int h, int w, int is_1d) {
        if (!name || c <= 0 || h <= 0 || w <= 0) return fail("add_input: bad arguments");
        const bool one_d = is_1d || h == 1;
        if (!one_d && w % 4 != 0) return fail("add_input: image width must be a multiple of 4");
        if (!nodes.empty()) return fail("add_input: the graph already has its input");
        is_2d = !one_d;
        GraphNode n;
        n.kind = GraphNode::INPUT; n.name = name; n.outs = {name}; n.cin = n.cout = (uint32_t)c; n.width = (uint32_t)w; n.height = (uint32_t)h;
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

    // k x k convolution of an image graph (k = 1 or 3, stride 1 or 2, pad = k / 2); weights FP16 [cout][cin][kh][kw]
    bool add_conv(const char *name, const char *in, const char *out, int cin, int cout, int kh, int kw, int stride, int pad, int act,
                  std::vector<uint16_t> &&w, const float *bias_f32, const char *residual) {
        if (!is_2d) return fail("add_conv2d: spatial convolutions need a 2-D image input");
        if (!((kh == 1 && kw == 1 && pad == 0) || (kh == 3 && kw == 3 && pad == 1)) || (stride != 1 && stride != 2))
            return fail("add_conv2d: supported windows are 1x1 (pad 0) and 3x3 (pad 1), stride 1 or 2");
        if (!add_linear(name, in, out, cin * kh * kw, cout, act, std::move(w), bias_f32, residual)) return false;
        GraphNode &n = nodes.back();
        n.cin = (uint32_t)cin; n.kh = (uint32_t)kh; n.kw = (uint32_t)kw; n.stride = (uint32_t)stride; n.pad = (uint32_t)pad;
        return true;
    }
    bool add_pool(const char *name, const char *in, const char *out, int k, int stride, int pad) {
        if (!is_2d) return fail("add_maxpool: needs a 2-D image input");
        if (!name || !in || !out || !((k == 2 && stride == 2 && pad == 0) || (k == 5 && stride == 1 && pad == 2)))
            return fail("add_maxpool: supported windows are 2x2 / stride 2 / pad 0 and 5x5 / stride 1 / pad 2");
        GraphNode n;
        n.kind = GraphNode::MAXPOOL; n.name = name; n.ins = {in}; n.outs = {out}; n.kh = n.kw = (uint32_t)k; n.stride = (uint32_t)stride; n.pad = (uint32_t)pad;
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }
    bool add_upsample(const char *name, const char *in, const char *out) {
        if (!is_2d) return fail("add_upsample2x: needs a 2-D image input");
        if (!name || !in || !out) return fail("add_upsample2x: bad arguments");
        GraphNode n;
        n.kind = GraphNode::UPSAMPLE; n.name = name; n.ins = {in}; n.outs = {out};
        nodes.push_back(std::move(n));
        compiled = false;
        return true;
    }
    // 2x2 / stride-2 transposed convolution; weights FP16 [cout][cin][4] (phase q = 2 * row parity + column parity)
    bool add_upconv(const char *name, const char *in, const char *out, int cin, int cout, std::vector<uint16_t> &&w, const float *bias_f32) {
        if (!is_2d) return fail("add_upconv2x2: needs a 2-D image input");
        if (!name || !in || !out || cin <= 0 || cout <= 0 || w.size() != (size_t)cin * cout * 4u) return fail("add_upconv2x2: bad arguments");
        GraphNode n;
        n.kind = GraphNode::UPCONV; n.name = name; n.ins = {in}; n.outs = {out}; n.cin = (uint32_t)cin; n.cout = (uint32_t)cout; n.w_f16 = std::move(w);
        n.bias_f16.assign((size_t)cout, 0);
        if (bias_f32) for (int i = 0; i < cout; ++i) n.bias_f16[i] = float_to_half(bias_f32[i]);
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
        if (is_2d) return compile_2d();
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

    // ---- 2-D image graphs -------------------------------------------------------------------------------
    // Every tensor [C][H][W] is C planes in the layout of its resolution (Layout2D). A convolution is one wave whose
    // gather offset of synapse (channel ch, tap ky, kx) is plane(ch) + (1 + dy) * W_pad + (1 + dx) relative to the tile
    // anchors, synapse order ch * taps + ky * kw + kx (the order of [cout][cin][kh][kw] weights). A stride-2 convolution
    // first splits its input into the four pixel-parity planes of every channel at half resolution (space-to-depth), which
    // turns tap (ky, kx) into a stride-1 tap on plane 4 ch + 2 py + px with dy = -1 for ky == 0 (else 0), py = 0 for ky == 1
    // (else 1), and the same along x. A 2x2 transposed convolution is a 1x1 wave producing the planes q * cout + c of the four
    // output phases at input resolution, followed by the scatter into the double-resolution tensor.
    bool compile_2d() {
        struct Shape { uint32_t c = 0, h = 0, w = 0; };
        std::map<std::string, Shape> shape;
        std::map<std::pair<uint32_t, uint32_t>, Layout2D> layouts;
        auto layout_of = [&](uint32_t h, uint32_t w) -> const Layout2D * {
            auto key = std::make_pair(h, w);
            auto it = layouts.find(key);
            if (it == layouts.end()) {
                Layout2D l;
                if (!l.init(h, w, std::max(1u, batch_size))) return nullptr;
                it = layouts.emplace(key, std::move(l)).first;
            }
            return &it->second;
        };
        // ---- shapes ----
        for (auto &n : nodes) {
            auto need = [&](const std::string &t) { return shape.count(t) != 0; };
            switch (n.kind) {
            case GraphNode::INPUT: shape[n.outs[0]] = {n.cout, n.height, n.width}; break;
            case GraphNode::LINEAR: {
                if (!need(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                const Shape in = shape[n.ins[0]];
                const uint32_t taps = n.kh * n.kw, cin = n.kh == 1 && n.kw == 1 && n.stride == 1 && n.w_f16.size() == (size_t)n.cin * n.cout ? n.cin : n.cin;
                if (in.c != cin) return fail("compile: " + n.name + " expects " + std::to_string(cin) + " input channels");
                if (n.w_f16.size() != (size_t)cin * taps * n.cout) return fail("compile: " + n.name + " has no weights");
                if (n.stride == 2 && (in.h % 2u || in.w % 8u)) return fail("compile: " + n.name + ": a stride-2 convolution needs an even height and a width that is a multiple of 8");
                const Shape out = {n.cout, in.h / n.stride, in.w / n.stride};
                if (!n.residual.empty()) {
                    if (!need(n.residual)) return fail("compile: residual tensor of " + n.name + " is missing");
                    const Shape r = shape[n.residual];
                    if (r.c < n.cout || r.h != out.h || r.w != out.w) return fail("compile: residual tensor of " + n.name + " has the wrong shape");
                }
                shape[n.outs[0]] = out;
                break;
            }
            case GraphNode::UPCONV: {
                if (!need(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                const Shape in = shape[n.ins[0]];
                if (in.c != n.cin) return fail("compile: " + n.name + " expects " + std::to_string(n.cin) + " input channels");
                shape[n.outs[0]] = {n.cout, in.h * 2u, in.w * 2u};
                break;
            }
            case GraphNode::MAXPOOL: {
                if (!need(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                const Shape in = shape[n.ins[0]];
                if (n.stride == 2 && (in.h % 2u || in.w % 8u)) return fail("compile: " + n.name + ": 2x2 pooling needs an even height and a width that is a multiple of 8");
                n.cin = n.cout = in.c;
                shape[n.outs[0]] = {in.c, in.h / n.stride, in.w / n.stride};
                break;
            }
            case GraphNode::UPSAMPLE: {
                if (!need(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                const Shape in = shape[n.ins[0]];
                n.cin = n.cout = in.c;
                shape[n.outs[0]] = {in.c, in.h * 2u, in.w * 2u};
                break;
            }
            case GraphNode::SPLIT:
                if (!need(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                for (auto &o : n.outs) shape[o] = shape[n.ins[0]];
                break;
            case GraphNode::SLICE: {
                if (!need(n.ins[0])) return fail("compile: unknown tensor " + n.ins[0]);
                const Shape in = shape[n.ins[0]];
                uint32_t sum = 0;
                for (size_t k = 0; k < n.outs.size(); ++k) {
                    const uint32_t part = n.slice_sizes.empty() ? in.c / (uint32_t)n.outs.size() : n.slice_sizes[k];
                    shape[n.outs[k]] = {part, in.h, in.w};
                    sum += part;
                }
                if (sum > in.c) return fail("compile: slice sizes exceed the tensor");
                break;
            }
            case GraphNode::CONCAT: {
                Shape acc;
                for (auto &i : n.ins) {
                    if (!need(i)) return fail("compile: unknown tensor " + i);
                    const Shape t = shape[i];
                    if (acc.c && (t.h != acc.h || t.w != acc.w)) return fail("compile: " + n.name + " joins tensors of different resolutions");
                    acc = {acc.c + t.c, t.h, t.w};
                }
                shape[n.outs[0]] = acc;
                break;
            }
            default: return fail("compile: node '" + n.name + "' belongs to 1-D token graphs");
            }
        }
        if (!shape.count(output_tensor)) output_tensor = nodes.back().outs[0];
        for (auto &kv : shape)
            if (!layout_of(kv.second.h, kv.second.w)) return fail("compile: tensor " + kv.first + " has no plane layout (width must be a multiple of 4; all frames of a plane at most 2^18 elements unless the width is a multiple of 64)");
        plan.batch_size = std::max(1u, batch_size);
        plan.is_2d = true;
        plan.layout.init(64, 1);
        plan.target = target;
        plan.reuse_canvas = reuse_canvas;

        // ---- canvas placement: one allocation per producing node (+ one for the polyphase planes of a stride-2 convolution
        // and one for the phase planes of a transposed convolution), by liveness with best-fit reuse when asked for ----
        struct Alloc { uint64_t len = 0, at = 0; size_t born = 0, dies = 0; };
        std::vector<Alloc> allocs;
        std::map<std::string, std::set<int>> aliases;
        std::vector<int> node_aid(nodes.size(), -1), node_tmp(nodes.size(), -1);
        auto planes_len = [&](uint32_t planes, const Layout2D *l) { return (((uint64_t)planes * l->channel_stride + 63u) & ~63ull) + 64u; };   // + slack: taps of the last tile
        for (size_t s = 0; s < nodes.size(); ++s) {
            auto &n = nodes[s];
            const bool produces2d = n.kind == GraphNode::INPUT || n.kind == GraphNode::LINEAR || n.kind == GraphNode::UPCONV || n.kind == GraphNode::MAXPOOL || n.kind == GraphNode::UPSAMPLE;
            if (produces2d) {
                const Shape o = shape[n.outs[0]];
                const uint32_t planes = (n.kind == GraphNode::LINEAR || n.kind == GraphNode::UPCONV) ? pad_cout(o.c) : o.c;
                node_aid[s] = (int)allocs.size();
                allocs.push_back({planes_len(planes, layout_of(o.h, o.w)), 0, s, s});
                aliases[n.outs[0]] = {node_aid[s]};
                if (n.kind == GraphNode::LINEAR && n.stride == 2) {
                    node_tmp[s] = (int)allocs.size();
                    allocs.push_back({planes_len(4u * n.cin, layout_of(o.h, o.w)), 0, s, s});
                } else if (n.kind == GraphNode::UPCONV) {
                    const Shape in = shape[n.ins[0]];
                    node_tmp[s] = (int)allocs.size();
                    allocs.push_back({planes_len(pad_cout(4u * n.cout), layout_of(in.h, in.w)), 0, s, s});
                }
            } else if (n.kind == GraphNode::CONCAT) {
                std::set<int> m;
                for (auto &i : n.ins) m.insert(aliases[i].begin(), aliases[i].end());
                aliases[n.outs[0]] = m;
            } else {
                for (auto &o : n.outs) aliases[o] = aliases[n.ins[0]];
            }
        }
        allocs[0].dies = nodes.size();
        for (int a : aliases[output_tensor]) allocs[a].dies = nodes.size();
        for (size_t s = 0; s < nodes.size(); ++s) {
            for (auto &i : nodes[s].ins) for (int a : aliases[i]) allocs[a].dies = std::max(allocs[a].dies, s);
            if (!nodes[s].residual.empty()) for (int a : aliases[nodes[s].residual]) allocs[a].dies = std::max(allocs[a].dies, s);
        }
        uint64_t peak = 0;
        if (!reuse_canvas) {
            for (auto &al : allocs) { al.at = peak; peak += al.len; }
        } else {
            // first fit over the regions that are dead when the allocation is born
            std::vector<size_t> order(allocs.size());
            for (size_t i = 0; i < order.size(); ++i) order[i] = i;
            std::vector<size_t> placed;
            for (size_t i : order) {
                uint64_t at = 0;
                bool moved = true;
                while (moved) {
                    moved = false;
                    for (size_t j : placed) {
                        const bool alive_together = !(allocs[j].dies < allocs[i].born || allocs[i].dies < allocs[j].born);
                        if (alive_together && at < allocs[j].at + allocs[j].len && allocs[j].at < at + allocs[i].len) { at = allocs[j].at + allocs[j].len; moved = true; }
                    }
                }
                allocs[i].at = at;
                placed.push_back(i);
                peak = std::max(peak, at + allocs[i].len);
            }
        }
        uint64_t canvas = (peak + 127u) / 128u * 128u;
        if (canvas > 0xffffffffull) return fail("compile: canvas exceeds 2^32 FP16 elements");
        plan.canvas_elems = std::max<uint64_t>(canvas, 128);

        // ---- command emission ----
        std::map<std::string, std::vector<uint64_t>> planes_of;     // tensor -> canvas offset of every channel's plane
        auto geom = [&](const Layout2D *l) { HostWave::Geom2D g; g.H = l->H; g.W = l->W; g.W_pad = l->W_pad; g.ch_stride = l->channel_stride; g.frames = l->frames; g.frame_stride = l->single_stride; return g; };
        auto contiguous2d = [&](const std::vector<uint64_t> &pl, const Layout2D *l) {
            for (size_t c = 1; c < pl.size(); ++c) if (pl[c] != pl[0] + (uint64_t)c * l->channel_stride) return false;
            return !pl.empty();
        };
        auto emit_halo_clear = [&](const std::string &name, uint64_t at, uint32_t planes, const Layout2D *l) {
            HostWave h;
            h.kind = 12; h.name = name + "_halo"; h.y_off = at; h.cout = h.logical_cout = planes; h.out2d = geom(l); h.in2d = h.out2d;
            h.h_out = l->H; h.w_out = l->W;
            plan.waves.push_back(std::move(h));
        };
        auto emit_wave = [&](const GraphNode &n, const std::string &wname, const std::vector<uint64_t> &in_planes, const Layout2D *l, uint32_t kh, uint32_t kw,
                             const std::vector<std::pair<int, int>> &tap_dydx, const std::vector<uint32_t> &tap_plane_mul, uint32_t cin, uint32_t cout_logical,
                             const std::vector<uint16_t> &w_rows /*[cout_logical][cin * taps]*/, const std::vector<uint16_t> &bias, int act, uint64_t dst,
                             const std::string &residual) -> bool {
            (void)kh; (void)kw; (void)tap_plane_mul;
            const uint32_t taps = (uint32_t)tap_dydx.size();
            HostWave w;
            w.name = wname;
            w.cin = cin; w.logical_cout = cout_logical; w.cout = pad_cout(cout_logical);
            w.fan_in_raw = cin * taps; w.fan_in = pad_fan_in(w.fan_in_raw);
            w.group = choose_group_size(w.cout, l->num_tiles, forced_group);
            w.act = act; w.has_bias = true;
            w.h_out = l->H; w.w_out = l->W;
            w.y_off = dst; w.src_off = in_planes[0];
            w.pitch2d = l->channel_stride; w.tile_mask = l->masked; w.tile_off_x = l->tile_off_x; w.tile_off_y = l->tile_off_y;
            if (!residual.empty()) {
                const auto &rp = planes_of[residual];
                if (!contiguous2d(rp, l) || rp.size() < cout_logical) return fail("compile: residual tensor of " + n.name + " is not stored as consecutive planes");
                w.has_residual = true;
                w.res_off = rp[0];
                const uint64_t end = w.res_off + (uint64_t)w.cout * l->channel_stride + 64u;
                if (end > plan.canvas_elems) plan.canvas_elems = (end + 127u) / 128u * 128u;
            }
            uint64_t lo = ~0ull, hi = 0;
            for (uint64_t pl : in_planes) { lo = std::min(lo, pl); hi = std::max(hi, pl); }
            if (hi + (uint64_t)l->channel_stride >= 0x70000000ull) w.x_base_off = lo & ~63ull;
            const uint32_t groups = w.cout / w.group;
            w.idx.assign((size_t)groups * w.fan_in, 0u);
            for (uint32_t g = 0; g < groups; ++g)
                for (uint32_t k = 0; k < w.fan_in_raw; ++k) {
                    // synapse k = ch * taps + tap; `in_planes` already lists the plane of every (ch, tap) when the taps pick planes
                    const uint32_t tap = k % taps;
                    const uint64_t plane = in_planes.size() == (size_t)cin * taps ? in_planes[k] : in_planes[k / taps];
                    w.idx[(size_t)g * w.fan_in + k] = (uint32_t)(l->tap(plane, tap_dydx[tap].first, tap_dydx[tap].second) - w.x_base_off);
                }
            w.bias.assign(w.cout, 0);
            std::copy(bias.begin(), bias.begin() + std::min<size_t>(bias.size(), cout_logical), w.bias.begin());
            std::vector<uint16_t> rm((size_t)w.cout * w.fan_in, 0);
            for (uint32_t j = 0; j < cout_logical; ++j)
                std::memcpy(&rm[(size_t)j * w.fan_in], &w_rows[(size_t)j * w.fan_in_raw], (size_t)w.fan_in_raw * 2);
            w.w_wmma.resize(rm.size());
            rowmajor_to_wmma(rm.data(), w.w_wmma.data(), w.cout, w.fan_in);
            const double gf = 2.0 * (double)w.fan_in_raw * (double)cout_logical * (double)l->H * (double)l->W / 1e9;
            w.gflops = gf * l->frames;
            plan.single_frame_gflops += gf;
            plan.total_gflops += gf * l->frames;
            plan.total_w_bytes += (uint64_t)w.cout * w.fan_in * 2;
            plan.total_idx_bytes += w.idx.size() * 4 + w.bias.size() * 2;
            plan.waves.push_back(std::move(w));
            return true;
        };
        for (size_t s = 0; s < nodes.size(); ++s) {
            auto &n = nodes[s];
            const bool produces2d = node_aid[s] >= 0;
            if (produces2d) {
                const Shape o = shape[n.outs[0]];
                const Layout2D *lo = layout_of(o.h, o.w);
                const uint64_t dst = allocs[node_aid[s]].at;
                std::vector<uint64_t> pl(o.c);
                for (uint32_t c = 0; c < o.c; ++c) pl[c] = dst + (uint64_t)c * lo->channel_stride;
                // recycled regions carry another tensor's pixels where this one has its halo
                if (reuse_canvas && n.kind != GraphNode::INPUT)
                    emit_halo_clear(n.name, dst, (n.kind == GraphNode::LINEAR || n.kind == GraphNode::UPCONV) ? pad_cout(o.c) : o.c, lo);
                if (n.kind == GraphNode::LINEAR) {
                    const auto &inp = planes_of[n.ins[0]];
                    const uint32_t taps = n.kh * n.kw;
                    std::vector<std::pair<int, int>> dydx;
                    std::vector<uint64_t> src = inp;
                    if (n.stride == 2) {
                        // space-to-depth into the half-resolution planes, then stride-1 taps on the parity planes
                        const Shape in = shape[n.ins[0]];
                        const Layout2D *li = layout_of(in.h, in.w);
                        if (!contiguous2d(inp, li)) return fail("compile: " + n.name + " (stride 2) reads a tensor that is not stored as consecutive planes");
                        const uint64_t tmp = allocs[node_tmp[s]].at;
                        if (reuse_canvas) emit_halo_clear(n.name + "_s2d", tmp, 4u * n.cin, lo);
                        HostWave sd;
                        sd.kind = 10; sd.name = n.name + "_s2d_2x2"; sd.src_off = inp[0]; sd.y_off = tmp; sd.cout = sd.logical_cout = n.cin; sd.cin = n.cin;
                        sd.in2d = geom(li); sd.out2d = geom(lo); sd.h_out = lo->H; sd.w_out = lo->W;
                        plan.waves.push_back(std::move(sd));
                        src.assign((size_t)n.cin * taps, 0);
                        for (uint32_t ch = 0; ch < n.cin; ++ch)
                            for (uint32_t ky = 0; ky < n.kh; ++ky)
                                for (uint32_t kx = 0; kx < n.kw; ++kx) {
                                    const uint32_t py = n.kh == 1 ? 0u : (ky == 1u ? 0u : 1u), pxx = n.kw == 1 ? 0u : (kx == 1u ? 0u : 1u);
                                    src[(size_t)ch * taps + ky * n.kw + kx] = tmp + (uint64_t)(4u * ch + 2u * py + pxx) * lo->channel_stride;
                                }
                        for (uint32_t ky = 0; ky < n.kh; ++ky)
                            for (uint32_t kx = 0; kx < n.kw; ++kx) dydx.push_back({n.kh == 1 ? 0 : (ky == 0 ? -1 : 0), n.kw == 1 ? 0 : (kx == 0 ? -1 : 0)});
                    } else {
                        for (uint32_t ky = 0; ky < n.kh; ++ky)
                            for (uint32_t kx = 0; kx < n.kw; ++kx) dydx.push_back({(int)ky - (int)(n.kh / 2u), (int)kx - (int)(n.kw / 2u)});
                    }
                    if (!emit_wave(n, n.name, src, lo, n.kh, n.kw, dydx, {}, n.cin, n.cout, n.w_f16, n.bias_f16, n.act, dst, n.residual)) return false;
                } else if (n.kind == GraphNode::UPCONV) {
                    const Shape in = shape[n.ins[0]];
                    const Layout2D *li = layout_of(in.h, in.w);
                    const auto &inp = planes_of[n.ins[0]];
                    const uint64_t tmp = allocs[node_tmp[s]].at;
                    if (reuse_canvas) emit_halo_clear(n.name + "_phases", tmp, pad_cout(4u * n.cout), li);
                    // rows q * cout + c of the phase wave: weights w[c][ci][q]
                    std::vector<uint16_t> wr((size_t)4u * n.cout * n.cin), br((size_t)4u * n.cout);
                    for (uint32_t q = 0; q < 4u; ++q)
                        for (uint32_t c = 0; c < n.cout; ++c) {
                            br[(size_t)q * n.cout + c] = n.bias_f16[c];
                            for (uint32_t ci = 0; ci < n.cin; ++ci) wr[((size_t)q * n.cout + c) * n.cin + ci] = n.w_f16[((size_t)c * n.cin + ci) * 4u + q];
                        }
                    if (!emit_wave(n, n.name + "_phases", inp, li, 1, 1, {{0, 0}}, {}, n.cin, 4u * n.cout, wr, br, ACT_NONE, tmp, "")) return false;
                    HostWave sc;
                    sc.kind = 11; sc.name = n.name + "_scatter"; sc.src_off = tmp; sc.y_off = dst; sc.cout = sc.logical_cout = n.cout; sc.cin = n.cin;
                    sc.in2d = geom(li); sc.out2d = geom(lo); sc.h_out = lo->H; sc.w_out = lo->W;
                    plan.waves.push_back(std::move(sc));
                } else if (n.kind == GraphNode::MAXPOOL || n.kind == GraphNode::UPSAMPLE) {
                    const Shape in = shape[n.ins[0]];
                    const Layout2D *li = layout_of(in.h, in.w);
                    const auto &inp = planes_of[n.ins[0]];
                    if (!contiguous2d(inp, li)) return fail("compile: " + n.name + " reads a tensor that is not stored as consecutive planes");
                    HostWave a;
                    a.kind = n.kind == GraphNode::UPSAMPLE ? 9 : (n.kh == 2 ? 7 : 8);
                    a.name = n.name; a.src_off = inp[0]; a.y_off = dst; a.cout = a.logical_cout = in.c; a.cin = in.c;
                    a.in2d = geom(li); a.out2d = geom(lo); a.h_out = lo->H; a.w_out = lo->W;
                    plan.waves.push_back(std::move(a));
                }
                planes_of[n.outs[0]] = std::move(pl);
            } else if (n.kind == GraphNode::SPLIT) {
                for (auto &o : n.outs) planes_of[o] = planes_of[n.ins[0]];
            } else if (n.kind == GraphNode::SLICE) {
                const auto &src = planes_of[n.ins[0]];
                size_t cur = 0;
                for (size_t k = 0; k < n.outs.size(); ++k) {
                    const size_t part = n.slice_sizes.empty() ? src.size() / n.outs.size() : n.slice_sizes[k];
                    planes_of[n.outs[k]] = std::vector<uint64_t>(src.begin() + cur, src.begin() + cur + part);
                    cur += part;
                }
            } else {
                std::vector<uint64_t> cat;
                for (auto &i : n.ins) cat.insert(cat.end(), planes_of[i].begin(), planes_of[i].end());
                planes_of[n.outs[0]] = std::move(cat);
            }
        }
        const Shape in0 = shape[nodes[0].outs[0]], outs = shape[output_tensor];
        const Layout2D *lin = layout_of(in0.h, in0.w), *lout = layout_of(outs.h, outs.w);
        const auto &out_planes = planes_of[output_tensor];
        if (!contiguous2d(out_planes, lout)) return fail("compile: the output tensor is not stored as consecutive planes");
        plan.input_off = allocs[0].at;
        plan.input_c = in0.c; plan.input_h = in0.h; plan.input_w = in0.w;
        plan.output_off = out_planes[0];
        plan.output_c = plan.logical_output_c = outs.c; plan.output_h = outs.h; plan.output_w = outs.w;
        plan.in2d = geom(lin); plan.out2d = geom(lout);
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
            static const char *types[] = {"K44_WAVE", "RMSNORM", "SWIGLU", "ROPE_GQA_ATTN", "DECODE_GQA_ATTN", "EMBEDDING", "ARGMAX", "MAXPOOL_2X2", "MAXPOOL_5X5",
                                          "UPSAMPLE_2X", "S2D_2X2", "SCATTER_UPCONV_2X2", "HALO_CLEAR"};
            std::snprintf(buf, sizeof buf,
                          "    {\"idx\": %zu, \"name\": \"%s\", \"type\": \"%s\", \"Cin\": %u, \"Cout\": %u, \"logical_Cout\": %u, "
                          "\"B\": %u, \"B_raw\": %u, \"S\": %u, \"act\": \"%s\", \"has_residual\": %s, \"has_self_read\": false, "
                          "\"subwave\": [0, 1], \"h_out\": %u, \"w_out\": %u, \"src_off\": %llu, \"y_off\": %llu, \"gflops\": %.6g}%s\n",
                          i, w.name.c_str(), types[w.kind >= 0 && w.kind <= 12 ? w.kind : 0], w.cin, w.cout, w.logical_cout, w.fan_in, w.fan_in_raw, w.group, act_name(w.act),
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
