// TCFFv1.0 container: writer and readers.
//
// Byte layout follows the reference container so that files are interchangeable
// (wavec/k44_tcff_io.hpp:100-300 writer, :319-428 reader). Little-endian throughout:
//   0   "II", u16 42, u32 offset of the first IFD
//   8   "TCFFv1.0", u32 alignment(256), u32 wave count, u32 canvas bytes, u32 flags,
//   32  u64 FNV-1a over bytes [8,32); zero padding to 256
//   per wave: weights (16x16-tile order) | pad | gather table | pad | bias | pad   (pad = to 256)
//             FNV-1a-64 over that whole span including the padding,
//             IFD: u16 count, 12-byte entries {u16 tag,u16 type,u32 count,u32 value-or-offset},
//             u32 next IFD, then 2-byte aligned external values, pad to 256.
// Every failure returns false with a message in `err`; nothing here terminates the process.
#pragma once
#include <cstdio>

#include "k44_host.hpp"

namespace k44b {

namespace tcff {
constexpr uint16_t T_ASCII = 2, T_SHORT = 3, T_LONG = 4, T_RATIONAL = 5;
constexpr uint16_t TAG_MAGIC = 0x8440, TAG_PARAMS = 0x8441, TAG_AUX = 0x8442, TAG_HASH = 0x8443, TAG_GEOM = 0x8444;
constexpr uint32_t MAGIC_WAVE = 0x45564157u;   // "WAVE"
constexpr uint32_t MAGIC_CANV = 0x564E4143u;   // "CANV" pages are skipped by readers
constexpr uint32_t FLAG_TRAILING_IFD_HASH = 1u, FLAG_HAS_CANVAS = 4u;
constexpr uint32_t ALIGN = 256u;

struct Out {
    std::vector<uint8_t> b;
    void u16(uint32_t v) { b.push_back((uint8_t)v); b.push_back((uint8_t)(v >> 8)); }
    void u32(uint32_t v) { u16(v & 0xffffu); u16(v >> 16); }
    void u64(uint64_t v) { u32((uint32_t)v); u32((uint32_t)(v >> 32)); }
    void bytes(const void *p, size_t n) { const uint8_t *q = (const uint8_t *)p; b.insert(b.end(), q, q + n); }
    void set32(size_t at, uint32_t v) { for (int i = 0; i < 4; ++i) b[at + i] = (uint8_t)(v >> (8 * i)); }
    void align(uint32_t a) { b.resize((b.size() + a - 1) / a * a, 0); }
    uint32_t pos() const { return (uint32_t)b.size(); }
};

inline uint32_t rd16(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }
inline uint32_t rd32(const uint8_t *p) { return rd16(p) | (rd16(p + 2) << 16); }
inline uint64_t rd64(const uint8_t *p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

inline bool slurp(const char *path, std::vector<uint8_t> &buf, std::string &err) {
    FILE *f = std::fopen(path, "rb");
    if (!f) { err = std::string("cannot open ") + path; return false; }
    std::fseek(f, 0, SEEK_END);
    long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    if (n < 0) { std::fclose(f); err = "cannot size file"; return false; }
    buf.resize((size_t)n);
    const bool ok = n == 0 || std::fread(buf.data(), 1, (size_t)n, f) == (size_t)n;
    std::fclose(f);
    if (!ok) err = "short read";
    return ok;
}
}  // namespace tcff

// One parsed wave page (views into the file buffer).
struct TcffWaveView {
    std::vector<uint32_t> params;   // tag 0x8441: Cin,Cout,B,S,weight_bits,3,act,has_residual,h_out,w_out
    std::vector<uint32_t> aux;      // tag 0x8442: w_off,w_bytes,idx_off,idx_bytes,bias_off,bias_bytes,src_off,y_off,start,end,res_off
    std::vector<uint32_t> geom;     // tag 0x8444 (optional)
    uint64_t hash = 0;
};

struct TcffView {
    uint32_t canvas_bytes = 0, flags = 0, num_waves = 0;
    std::vector<TcffWaveView> waves;
};

inline bool tcff_serialize(const HostPlan &plan, const char *prefix, bool include_geometry,
                           std::vector<uint8_t> &out_bytes, std::string &err) {
    using namespace tcff;
    const char *pfx = (prefix && prefix[0]) ? prefix : "K44Model";
    // only waves have pages; element-wise / attention commands carry no tensors worth storing (an RMSNorm scale that
    // was not folded into the next waves stays with the graph)
    std::vector<const HostWave *> ws;
    for (const auto &w : plan.waves) if (w.kind == 0) ws.push_back(&w);
    const uint32_t nw = (uint32_t)ws.size();
    uint64_t need = 4096;
    for (const HostWave *w : ws) need += (uint64_t)w->cout * w->fan_in * 2 + w->idx.size() * 4 + w->cout * 2 + 4096;
    if (need >= 0xffffffffull) { err = "plan too large for a TCFFv1.0 file (32-bit offsets)"; return false; }
    Out o;
    o.b.reserve((size_t)need);
    o.bytes("II", 2); o.u16(42); o.u32(0);
    o.bytes("TCFFv1.0", 8);
    o.u32(ALIGN); o.u32(nw); o.u32((uint32_t)(plan.canvas_elems * 2ull)); o.u32(FLAG_TRAILING_IFD_HASH);
    o.u64(fnv1a64(o.b.data() + 8, 24));
    o.align(ALIGN);
    size_t link = 4;
    for (uint32_t wi = 0; wi < nw; ++wi) {
        const HostWave &w = *ws[wi];
        if (w.w_wmma.size() != (size_t)w.cout * w.fan_in) { err = "wave " + w.name + " has no host weights"; return false; }
        const uint32_t start = o.pos();
        const uint32_t w_off = o.pos(), w_bytes = (uint32_t)(w.w_wmma.size() * 2);
        o.bytes(w.w_wmma.data(), w_bytes); o.align(ALIGN);
        const uint32_t i_off = o.pos(), i_bytes = (uint32_t)(w.idx.size() * 4);
        for (uint32_t v : w.idx) o.u32(v);
        o.align(ALIGN);
        const uint32_t b_off = o.pos(), b_bytes = (uint32_t)(w.bias.size() * 2);
        for (uint16_t v : w.bias) o.u16(v);
        o.align(ALIGN);
        const uint32_t end = o.pos();
        const uint64_t h = fnv1a64(o.b.data() + start, end - start);

        const uint32_t ifd = o.pos();
        o.set32(link, ifd);
        const uint32_t ntags = 21u + (include_geometry ? 1u : 0u);
        const uint32_t ext0 = ifd + 2u + ntags * 12u + 4u;
        Out ext;
        auto put = [&](const void *p, size_t n) { if (ext.b.size() & 1u) ext.b.push_back(0); uint32_t at = ext0 + ext.pos(); ext.bytes(p, n); return at; };
        auto put32 = [&](std::initializer_list<uint32_t> v) { Out t; for (uint32_t x : v) t.u32(x); return put(t.b.data(), t.b.size()); };

        char page[128], desc[320];
        std::snprintf(page, sizeof page, "%s_Wave_%03u_%ux%u_S%u", pfx, wi, w.fan_in, w.cout, w.group);
        std::snprintf(desc, sizeof desc,
                      "TCFF %s Wave %u/%u | Cin=%u Cout=%u(log=%u) B=%u S=%u Act=%s Res=%d | W=0x%x Idx=0x%x Bias=0x%x | FNV1a64=0x%016llx",
                      pfx, wi, nw, w.cin, w.cout, w.logical_cout, w.fan_in, w.group,
                      w.act <= ACT_LEAKY_RELU ? act_name(w.act) : "NONE", (int)w.has_residual, w_off, i_off, b_off,
                      (unsigned long long)h);
        const uint32_t desc_len = (uint32_t)std::strlen(desc) + 1, page_len = (uint32_t)std::strlen(page) + 1;
        const uint32_t desc_at = put(desc, desc_len);
        const uint32_t page_at = put(page, page_len);
        const uint32_t rat_at = put32({1u, 1u});
        const uint32_t par_at = put32({w.cin, w.cout, w.fan_in, w.group, w.weight_bits, 3u, (uint32_t)w.act,
                                       (uint32_t)w.has_residual, w.h_out, w.w_out});
        const uint32_t aux_at = put32({w_off, w_bytes, i_off, i_bytes, b_off, b_bytes, (uint32_t)w.src_off,
                                       (uint32_t)w.y_off, start, end, (uint32_t)w.res_off});
        const uint32_t hash_at = put32({(uint32_t)h, (uint32_t)(h >> 32)});
        uint32_t geom_at = 0;
        if (include_geometry) {
            const uint32_t tokens = std::max(1u, w.w_out);
            geom_at = put32({tokens > 1u ? 2u : 1u, tokens, w.logical_cout, 1u, 1u, 1u, plan.layout.channel_stride, 1u, 1u, 0u});
        }
        struct E { uint16_t tag, type; uint32_t count, value; };
        std::vector<E> es = {
            {254, T_LONG, 1, 2u}, {256, T_LONG, 1, w.fan_in}, {257, T_LONG, 1, w.cout}, {258, T_SHORT, 1, w.weight_bits},
            {259, T_SHORT, 1, 1u}, {262, T_SHORT, 1, 1u}, {266, T_SHORT, 1, 1u}, {270, T_ASCII, desc_len, desc_at},
            {273, T_LONG, 1, w_off}, {277, T_SHORT, 1, 1u}, {278, T_LONG, 1, w.cout}, {279, T_LONG, 1, w_bytes},
            {282, T_RATIONAL, 1, rat_at}, {283, T_RATIONAL, 1, rat_at}, {285, T_ASCII, page_len, page_at},
            {297, T_SHORT, 2, wi | (nw << 16)}, {339, T_SHORT, 1, 3u}, {TAG_MAGIC, T_LONG, 1, MAGIC_WAVE},
            {TAG_PARAMS, T_LONG, 10, par_at}, {TAG_AUX, T_LONG, 11, aux_at}, {TAG_HASH, T_LONG, 2, hash_at}};
        if (include_geometry) es.push_back({TAG_GEOM, T_LONG, 10, geom_at});
        o.u16((uint32_t)es.size());
        for (const E &e : es) { o.u16(e.tag); o.u16(e.type); o.u32(e.count); o.u32(e.value); }
        link = o.b.size();
        o.u32(0);
        o.bytes(ext.b.data(), ext.b.size());
        o.align(ALIGN);
    }
    out_bytes.swap(o.b);
    return true;
}

inline bool tcff_save(const HostPlan &plan, const char *path, const char *prefix, bool include_geometry, std::string &err) {
    std::vector<uint8_t> bytes;
    if (!tcff_serialize(plan, prefix, include_geometry, bytes, err)) return false;
    FILE *f = std::fopen(path, "wb");
    if (!f) { err = std::string("cannot create ") + path; return false; }
    const bool ok = std::fwrite(bytes.data(), 1, bytes.size(), f) == bytes.size();
    std::fclose(f);
    if (!ok) err = "short write";
    return ok;
}

// Parse and verify a container held in memory. Every offset is range-checked against the buffer
// (the reference reader trusts them); both hash levels are verified.
inline bool tcff_parse(const std::vector<uint8_t> &buf, TcffView &view, std::string &err) {
    using namespace tcff;
    const size_t n = buf.size();
    if (n < 256) { err = "file shorter than the 256-byte header"; return false; }
    const uint8_t *d = buf.data();
    if (d[0] != 'I' || d[1] != 'I' || rd16(d + 2) != 42u) { err = "not a little-endian TIFF header"; return false; }
    if (std::memcmp(d + 8, "TCFFv1.0", 8) != 0) { err = "TCFFv1.0 magic missing"; return false; }
    if (rd64(d + 32) != fnv1a64(d + 8, 24)) { err = "master header hash mismatch"; return false; }
    view.num_waves = rd32(d + 20);
    view.canvas_bytes = rd32(d + 24);
    view.flags = rd32(d + 28);
    view.waves.clear();
    uint64_t ifd = rd32(d + 4);
    size_t guard = 0;
    while (ifd != 0) {
        if (++guard > 1000000 || ifd + 2 > n) { err = "IFD offset outside the file"; return false; }
        const uint32_t cnt = rd16(d + ifd);
        const uint64_t tail = ifd + 2 + (uint64_t)cnt * 12;
        if (tail + 4 > n) { err = "IFD table truncated"; return false; }
        uint32_t magic = 0, aux_at = 0, aux_n = 0, hash_at = 0, par_at = 0, par_n = 0, geo_at = 0, geo_n = 0;
        for (uint32_t i = 0; i < cnt; ++i) {
            const uint8_t *e = d + ifd + 2 + (uint64_t)i * 12;
            const uint32_t tag = rd16(e), c = rd32(e + 4), v = rd32(e + 8);
            if (tag == TAG_MAGIC) magic = v;
            else if (tag == TAG_AUX) { aux_at = v; aux_n = c; }
            else if (tag == TAG_HASH) hash_at = v;
            else if (tag == TAG_PARAMS) { par_at = v; par_n = c; }
            else if (tag == TAG_GEOM) { geo_at = v; geo_n = c; }
        }
        const uint64_t next = rd32(d + tail);
        if (magic == MAGIC_CANV) { ifd = next; continue; }
        if (aux_at == 0 || aux_n < 10 || hash_at == 0) { err = "wave page without aux/hash tags"; return false; }
        if ((uint64_t)aux_at + (uint64_t)aux_n * 4 > n || (uint64_t)hash_at + 8 > n ||
            (uint64_t)par_at + (uint64_t)par_n * 4 > n || (uint64_t)geo_at + (uint64_t)geo_n * 4 > n) {
            err = "tag value outside the file"; return false;
        }
        TcffWaveView wv;
        for (uint32_t i = 0; i < aux_n; ++i) wv.aux.push_back(rd32(d + aux_at + 4 * i));
        for (uint32_t i = 0; i < par_n; ++i) wv.params.push_back(rd32(d + par_at + 4 * i));
        for (uint32_t i = 0; i < geo_n; ++i) wv.geom.push_back(rd32(d + geo_at + 4 * i));
        wv.hash = rd64(d + hash_at);
        const uint64_t s = wv.aux[8], e = wv.aux[9];
        if (s > e || e > n) { err = "wave data span outside the file"; return false; }
        for (int k = 0; k < 6; k += 2)
            if ((uint64_t)wv.aux[k] + wv.aux[k + 1] > n) { err = "wave block outside the file"; return false; }
        if (fnv1a64(d + s, (size_t)(e - s)) != wv.hash) {
            err = "wave " + std::to_string(view.waves.size()) + " hash mismatch"; return false;
        }
        view.waves.push_back(std::move(wv));
        ifd = next;
    }
    return true;
}

// Fill an already-compiled plan from a file — the contract of the reference's
// load_weights_from_tcff (wavec/k44_tcff_io.hpp:319-428): weights and bias are always taken, the
// gather table only when batch_size == 1, the file's canvas size equals the plan's and the table
// size matches. The file must hold at least as many wave pages as the plan has waves.
inline bool tcff_load_into(HostPlan &plan, const char *path, std::string &err) {
    std::vector<uint8_t> buf;
    TcffView view;
    if (!tcff::slurp(path, buf, err) || !tcff_parse(buf, view, err)) return false;
    std::vector<HostWave *> ws;
    for (auto &w : plan.waves) if (w.kind == 0) ws.push_back(&w);
    if (view.waves.size() < ws.size()) { err = "file has fewer wave pages than the plan"; return false; }
    const bool take_idx = plan.batch_size == 1u && plan.canvas_elems * 2ull == (uint64_t)view.canvas_bytes;
    for (size_t i = 0; i < ws.size(); ++i) {
        HostWave &w = *ws[i];
        const auto &a = view.waves[i].aux;
        const size_t want_w = (size_t)w.cout * w.fan_in * 2;
        w.w_wmma.assign(std::max(want_w, (size_t)a[1]) / 2, 0);
        std::memcpy(w.w_wmma.data(), buf.data() + a[0], std::min(want_w, (size_t)a[1]));
        w.w_wmma.resize(want_w / 2);
        if (take_idx && a[3] == w.idx.size() * 4)
            for (size_t k = 0; k < w.idx.size(); ++k) w.idx[k] = tcff::rd32(buf.data() + a[2] + 4 * k);
        w.bias.assign(w.cout, 0);
        const size_t nb = std::min((size_t)w.cout, (size_t)a[5] / 2);
        for (size_t k = 0; k < nb; ++k) w.bias[k] = (uint16_t)tcff::rd16(buf.data() + a[4] + 2 * k);
    }
    return true;
}

// Rebuild a pure-wave 1-D plan from the file alone (no graph needed): dimensions and offsets come
// from tags 0x8441 / 0x8442 / 0x8444. The pitch is taken from the geometry tag; without it the
// caller must supply one. Input/output regions default to the first wave's source and the last
// wave's destination.
inline bool tcff_to_plan(const char *path, uint32_t pitch_hint, HostPlan &plan, std::string &err) {
    std::vector<uint8_t> buf;
    TcffView view;
    if (!tcff::slurp(path, buf, err) || !tcff_parse(buf, view, err)) return false;
    if (view.waves.empty()) { err = "file holds no wave pages"; return false; }
    plan = HostPlan();
    uint32_t pitch = pitch_hint;
    for (const auto &wv : view.waves)
        if (wv.geom.size() >= 10 && wv.geom[6] >= 64) pitch = wv.geom[6];
    if (pitch == 0 || pitch % 64 != 0) { err = "no usable row pitch (geometry tag missing and no hint given)"; return false; }
    plan.layout.init(pitch, 1);
    plan.layout.width = view.waves.back().params.size() >= 10 ? std::max(1u, view.waves.back().params[9]) : pitch;
    plan.canvas_elems = view.canvas_bytes / 2;
    for (size_t i = 0; i < view.waves.size(); ++i) {
        const auto &wv = view.waves[i];
        if (wv.params.size() < 10) { err = "wave parameter tag too short"; return false; }
        HostWave w;
        w.name = "wave" + std::to_string(i);
        w.cin = wv.params[0]; w.cout = wv.params[1]; w.fan_in = wv.params[2]; w.group = wv.params[3];
        w.weight_bits = wv.params[4]; w.act = (int)wv.params[6]; w.has_residual = wv.params[7] != 0;
        w.h_out = wv.params[8]; w.w_out = wv.params[9];
        w.logical_cout = wv.geom.size() >= 3 ? wv.geom[2] : w.cout;
        w.fan_in_raw = std::min(w.fan_in, w.cin ? w.cin : w.fan_in);
        w.src_off = wv.aux[6]; w.y_off = wv.aux[7]; w.res_off = wv.aux.size() > 10 ? wv.aux[10] : 0;
        if (w.group == 0 || w.cout % w.group || w.fan_in % 8 || w.cout % 16) { err = "inconsistent wave dimensions"; return false; }
        if ((uint64_t)wv.aux[1] != (uint64_t)w.cout * w.fan_in * 2 || (uint64_t)wv.aux[3] != (uint64_t)(w.cout / w.group) * w.fan_in * 4 ||
            (uint64_t)wv.aux[5] < (uint64_t)w.cout * 2) { err = "block sizes do not match the wave dimensions"; return false; }
        w.w_wmma.resize((size_t)w.cout * w.fan_in);
        std::memcpy(w.w_wmma.data(), buf.data() + wv.aux[0], w.w_wmma.size() * 2);
        w.idx.resize((size_t)(w.cout / w.group) * w.fan_in);
        for (size_t k = 0; k < w.idx.size(); ++k) w.idx[k] = tcff::rd32(buf.data() + wv.aux[2] + 4 * k);
        w.bias.resize(w.cout);
        for (size_t k = 0; k < w.bias.size(); ++k) w.bias[k] = (uint16_t)tcff::rd16(buf.data() + wv.aux[4] + 2 * k);
        plan.total_w_bytes += (uint64_t)w.cout * w.fan_in * 2;
        plan.total_idx_bytes += w.idx.size() * 4 + w.bias.size() * 2;
        plan.waves.push_back(std::move(w));
    }
    const HostWave &first = plan.waves.front(), &last = plan.waves.back();
    plan.input_off = first.src_off; plan.input_c = first.cin; plan.input_w = plan.layout.width;
    plan.output_off = last.y_off; plan.output_c = last.cout; plan.logical_output_c = last.logical_cout;
    plan.output_w = plan.layout.width;
    return true;
}

}  // namespace k44b
