// overlay.cu -- the safetensors overlay of NVFP4 triples: writer, reader and the family tables (host code).
//
// Wire format of the reference's requant tool (tools/requant_dense_nvfp4.py): for every selected bf16
// tensor `<stem>.weight` three tensors `<stem>.weight_packed` (U8 [N, K/2]), `<stem>.weight_scale`
// (F8_E4M3 [N, K/16]) and `<stem>.weight_global_scale` (F32 [1]) in shards `overlay-%05d.safetensors`
// (ShardWriter, :123-152: 8-byte little-endian header length, compact JSON header in insertion order
// padded with spaces so that the data starts on a 16-byte boundary, every tensor padded to 16 bytes),
// plus `model.safetensors.index.json` (:238-239).  The writer here produces the same bytes, so that a
// GPU-side requantisation (b200_nvfp4_quantize) can emit an overlay the reference's loader
// (include/safetensors.h:54-113, include/weight_store.h:23-33) takes as is; the reader maps such an
// overlay back into host pointers.  Which tensors belong in an overlay is decided by the tool's family
// tables (:76-113), restated below.
#include "b200_internal.h"
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <regex>
#include <string>
#include <vector>

namespace {

// ---- family tables (reference tools/requant_dense_nvfp4.py:76-113) --------------------------------
struct Family { const char* name; const char* pattern; };
const Family GLM5[] = {
    {"kda_qkv", R"(layers\.\d+\.self_attn\.[qkv]_proj\.weight$)"},
    {"o_proj", R"(layers\.\d+\.self_attn\.o_proj\.weight$)"},
    {"kda_gates", R"(layers\.\d+\.self_attn\.(f_a|f_b|g_a|g_b|b)_proj\.weight$)"},
    {"mla", R"(layers\.\d+\.self_attn\.(q_a_proj|q_b_proj|kv_a_proj_with_mqa)\.weight$)"},
    {"indexer", R"(layers\.\d+\.self_attn\.indexer\.(wq_b|wk|weights_proj)\.weight$|index_kpool_compress_gate$)"},
    {"dense_mlp", R"(layers\.\d+\.mlp\.(gate|up|down)_proj\.weight$)"},
    {"lm_head", R"(^lm_head\.weight$)"},
};
const char* GLM5_DEFAULT = "kda_qkv,o_proj,lm_head,dense_mlp,mla,indexer,kda_gates";
const Family MIMO[] = {
    {"o_proj", R"(^model\.layers\.\d+\.self_attn\.o_proj\.weight$)"},
    {"lm_head", R"(^lm_head\.weight$)"},
    {"mtp_o", R"(^model\.mtp\.layers\.\d+\.self_attn\.o_proj\.weight$)"},
};
const char* MIMO_DEFAULT = "o_proj";

std::string json_escape(const std::string& s) {
    std::string o;
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { o += '\\'; o += (char)c; }
        else if (c < 0x20 || c >= 0x7f) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += (char)c;
    }
    return o;
}

struct Shard {
    std::string path, header;                       // header: the JSON object's members so far, comma separated
    std::vector<std::pair<const void*, size_t>> parts;    // caller memory; copied out at flush
    std::vector<std::vector<unsigned char>> owned;  // copies of the tensors (the caller's buffers may go away)
    uint64_t off = 0;
};

}  // namespace

struct b200_overlay_writer {
    std::string dir;
    uint64_t shard_bytes = 0, written = 0;
    int shard_index = 0;
    Shard cur;
    std::vector<std::pair<std::string, std::string>> index;    // tensor name -> shard file, insertion order
};

static void shard_add(Shard& s, const std::string& name, const void* data, size_t bytes, const char* dtype, const std::vector<long>& shape) {
    const uint64_t pad = (16 - s.off % 16) % 16;
    if (pad) { s.owned.emplace_back(pad, (unsigned char)0); s.off += pad; }
    char buf[160];
    std::string sh;
    for (size_t i = 0; i < shape.size(); ++i) { snprintf(buf, sizeof buf, "%s%ld", i ? "," : "", shape[i]); sh += buf; }
    snprintf(buf, sizeof buf, "\":{\"dtype\":\"%s\",\"shape\":[%s],\"data_offsets\":[%llu,%llu]}", dtype, sh.c_str(),
             (unsigned long long)s.off, (unsigned long long)(s.off + bytes));
    if (!s.header.empty()) s.header += ',';
    s.header += '"'; s.header += json_escape(name); s.header += buf;
    s.owned.emplace_back(static_cast<const unsigned char*>(data), static_cast<const unsigned char*>(data) + bytes);
    s.off += bytes;
}

static int shard_flush(Shard& s) {
    std::string hdr = "{" + s.header + "}";
    hdr.append((16 - (8 + hdr.size()) % 16) % 16, ' ');     // the data starts 16-byte aligned
    FILE* f = fopen(s.path.c_str(), "wb");
    if (!f) { fprintf(stderr, "b200_nvfp4: cannot write %s\n", s.path.c_str()); return B200_EINVAL; }
    const uint64_t n = hdr.size();
    bool ok = fwrite(&n, 8, 1, f) == 1 && fwrite(hdr.data(), 1, hdr.size(), f) == hdr.size();
    for (const auto& b : s.owned) ok = ok && (b.empty() || fwrite(b.data(), 1, b.size(), f) == b.size());
    ok = fclose(f) == 0 && ok;
    s = Shard{};
    return ok ? B200_OK : B200_EINVAL;
}

static std::string shard_name(int i) { char b[64]; snprintf(b, sizeof b, "overlay-%05d.safetensors", i); return b; }

extern "C" int b200_overlay_writer_open(b200_overlay_writer** out, const char* dir, uint64_t shard_bytes) {
    if (!out || !dir) return B200_EINVAL;
    mkdir(dir, 0777);                                           // like os.makedirs(exist_ok=True) for one level
    b200_overlay_writer* w = new (std::nothrow) b200_overlay_writer();
    if (!w) return B200_ELIMIT;
    w->dir = dir; w->shard_bytes = shard_bytes ? shard_bytes : (2ull << 30);
    w->cur.path = w->dir + "/" + shard_name(0);
    *out = w;
    return B200_OK;
}

extern "C" int b200_overlay_writer_add(b200_overlay_writer* w, const char* tensor_name, const uint8_t* packed,
                                       const uint8_t* scale, float gscale, int N, int K) {
    if (!w || !tensor_name || !packed || !scale || N < 1 || K < 16 || (K & 15)) return B200_EINVAL;
    std::string stem = tensor_name;
    const std::string suf = ".weight";
    if (stem.size() >= suf.size() && stem.compare(stem.size() - suf.size(), suf.size(), suf) == 0) stem.resize(stem.size() - suf.size());
    const size_t pb = (size_t)N * (K / 2), sb = (size_t)N * (K / 16);
    shard_add(w->cur, stem + ".weight_packed", packed, pb, "U8", {N, K / 2});
    shard_add(w->cur, stem + ".weight_scale", scale, sb, "F8_E4M3", {N, K / 16});
    shard_add(w->cur, stem + ".weight_global_scale", &gscale, 4, "F32", {1});
    const std::string file = shard_name(w->shard_index);
    for (const char* s3 : {".weight_packed", ".weight_scale", ".weight_global_scale"}) w->index.emplace_back(stem + s3, file);
    w->written += pb + sb + 4;
    if (w->cur.off >= w->shard_bytes) {
        if (int rc = shard_flush(w->cur)) return rc;
        w->cur.path = w->dir + "/" + shard_name(++w->shard_index);
    }
    return B200_OK;
}

extern "C" int b200_overlay_writer_close(b200_overlay_writer* w) {
    if (!w) return B200_EINVAL;
    int rc = B200_OK;
    if (!w->cur.header.empty()) rc = shard_flush(w->cur);
    // json.dump's default separators (", " and ": "), keys in insertion order (reference :238-239)
    std::string idx = "{\"metadata\": {\"total_size\": " + std::to_string(w->written) + "}, \"weight_map\": {";
    // a name written twice keeps its first position and its last value, as a Python dict does
    std::vector<std::pair<std::string, std::string>> uniq;
    std::map<std::string, size_t> pos;
    for (const auto& kv : w->index) {
        auto it = pos.find(kv.first);
        if (it == pos.end()) { pos[kv.first] = uniq.size(); uniq.push_back(kv); } else uniq[it->second].second = kv.second;
    }
    for (size_t i = 0; i < uniq.size(); ++i)
        idx += std::string(i ? ", " : "") + "\"" + json_escape(uniq[i].first) + "\": \"" + uniq[i].second + "\"";
    idx += "}}";
    FILE* f = fopen((w->dir + "/model.safetensors.index.json").c_str(), "wb");
    if (!f || fwrite(idx.data(), 1, idx.size(), f) != idx.size()) rc = B200_EINVAL;
    if (f) fclose(f);
    delete w;
    return rc;
}

// ---- family selection -----------------------------------------------------------------------------
// Index of the first selected family (in the order of `families_csv`) whose pattern matches, -1 if none
// or if the tensor is excluded (vision tower, embeddings); -2 for an unknown arch or family.
extern "C" int b200_overlay_family(const char* arch, const char* families_csv, const char* tensor_name) {
    if (!arch || !tensor_name) return -2;
    const Family* tab; int n; const char* dflt;
    if (!strcmp(arch, "glm5")) { tab = GLM5; n = (int)(sizeof GLM5 / sizeof GLM5[0]); dflt = GLM5_DEFAULT; }
    else if (!strcmp(arch, "mimo")) { tab = MIMO; n = (int)(sizeof MIMO / sizeof MIMO[0]); dflt = MIMO_DEFAULT; }
    else return -2;
    const std::string name = tensor_name, sel = families_csv && *families_csv ? families_csv : dflt;
    if (name.find(".visual.") != std::string::npos || name.rfind("visual.", 0) == 0 || name.find("embed_tokens") != std::string::npos) return -1;
    int idx = 0;
    for (size_t a = 0; a <= sel.size();) {
        size_t b = sel.find(',', a);
        if (b == std::string::npos) b = sel.size();
        std::string f = sel.substr(a, b - a);
        while (!f.empty() && f.front() == ' ') f.erase(f.begin());
        while (!f.empty() && f.back() == ' ') f.pop_back();
        a = b + 1;
        if (f.empty()) continue;
        const Family* hit = nullptr;
        for (int i = 0; i < n; ++i) if (f == tab[i].name) hit = &tab[i];
        if (!hit) return -2;
        if (std::regex_search(name, std::regex(hit->pattern, std::regex::ECMAScript))) return idx;
        ++idx;
    }
    return -1;
}

// ---- reader ---------------------------------------------------------------------------------------
namespace {
struct Mapped { int fd = -1; const unsigned char* base = nullptr; size_t size = 0; };
struct Tens { const unsigned char* data; size_t bytes; std::string dtype; std::vector<long> shape; };

// Minimal JSON walker for a safetensors header: an object of name -> {dtype, shape, data_offsets}.
struct Json {
    const char* p; const char* end;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
    std::string str() {
        ws(); std::string s;
        if (p >= end || *p != '"') return s;
        for (++p; p < end && *p != '"'; ++p) {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                if (*p == 'u' && p + 4 < end) { s += (char)strtol(std::string(p + 1, p + 5).c_str(), nullptr, 16); p += 4; }
                else s += *p;
            } else s += *p;
        }
        if (p < end) ++p;
        return s;
    }
    double num() { ws(); char* e; const double v = strtod(p, &e); p = e; return v; }
    void skip() {
        ws();
        if (p >= end) return;
        if (*p == '"') { str(); }
        else if (*p == '{') { ++p; if (eat('}')) return; do { str(); eat(':'); skip(); } while (eat(',')); eat('}'); }
        else if (*p == '[') { ++p; if (eat(']')) return; do { skip(); } while (eat(',')); eat(']'); }
        else while (p < end && *p != ',' && *p != '}' && *p != ']') ++p;
    }
};
}  // namespace

struct b200_overlay {
    std::vector<Mapped> files;
    std::map<std::string, Tens> tensors;
};

extern "C" int b200_overlay_close(b200_overlay* o) {
    if (!o) return B200_EINVAL;
    for (Mapped& m : o->files) { if (m.base) munmap((void*)m.base, m.size); if (m.fd >= 0) close(m.fd); }
    delete o;
    return B200_OK;
}

extern "C" int b200_overlay_open(b200_overlay** out, const char* dir) {
    if (!out || !dir) return B200_EINVAL;
    b200_overlay* o = new (std::nothrow) b200_overlay();
    if (!o) return B200_ELIMIT;
    for (int i = 0;; ++i) {
        const std::string path = std::string(dir) + "/" + shard_name(i);
        Mapped m;
        m.fd = open(path.c_str(), O_RDONLY);
        if (m.fd < 0) break;
        struct stat sb;
        if (fstat(m.fd, &sb) != 0 || sb.st_size < 8) { close(m.fd); b200_overlay_close(o); return B200_EINVAL; }
        m.size = (size_t)sb.st_size;
        m.base = static_cast<const unsigned char*>(mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, m.fd, 0));
        if (m.base == MAP_FAILED) { close(m.fd); b200_overlay_close(o); return B200_EINVAL; }
        o->files.push_back(m);
        uint64_t hlen; memcpy(&hlen, m.base, 8);
        if (8 + hlen > m.size) { b200_overlay_close(o); return B200_EINVAL; }
        const unsigned char* data = m.base + 8 + hlen;
        Json j{reinterpret_cast<const char*>(m.base) + 8, reinterpret_cast<const char*>(m.base) + 8 + hlen};
        if (!j.eat('{')) { b200_overlay_close(o); return B200_EINVAL; }
        if (j.eat('}')) continue;
        do {
            const std::string name = j.str(); j.eat(':');
            if (name == "__metadata__") { j.skip(); continue; }
            Tens t{}; long o0 = 0, o1 = 0;
            j.eat('{');
            do {
                const std::string key = j.str(); j.eat(':');
                if (key == "dtype") t.dtype = j.str();
                else if (key == "shape") { j.eat('['); if (!j.eat(']')) { do { t.shape.push_back((long)j.num()); } while (j.eat(',')); j.eat(']'); } }
                else if (key == "data_offsets") { j.eat('['); o0 = (long)j.num(); j.eat(','); o1 = (long)j.num(); j.eat(']'); }
                else j.skip();
            } while (j.eat(','));
            j.eat('}');
            if (o0 < 0 || o1 < o0 || 8 + hlen + (uint64_t)o1 > m.size) { b200_overlay_close(o); return B200_EINVAL; }
            t.data = data + o0; t.bytes = (size_t)(o1 - o0);
            o->tensors[name] = t;
        } while (j.eat(','));
    }
    if (o->files.empty()) { b200_overlay_close(o); return B200_EINVAL; }
    *out = o;
    return B200_OK;
}

extern "C" int b200_overlay_count(const b200_overlay* o) { return o ? (int)(o->tensors.size() / 3) : 0; }

// The triple of `<stem>.weight` (the name with or without the ".weight" suffix).  Pointers are HOST pointers
// into the mapped shard, valid until b200_overlay_close; packed and scale are 16-byte aligned in the file.
extern "C" int b200_overlay_find(const b200_overlay* o, const char* tensor_name, b200_overlay_entry* out) {
    if (!o || !tensor_name || !out) return B200_EINVAL;
    std::string stem = tensor_name;
    const std::string suf = ".weight";
    if (stem.size() >= suf.size() && stem.compare(stem.size() - suf.size(), suf.size(), suf) == 0) stem.resize(stem.size() - suf.size());
    auto p = o->tensors.find(stem + ".weight_packed"), s = o->tensors.find(stem + ".weight_scale"), g = o->tensors.find(stem + ".weight_global_scale");
    if (p == o->tensors.end() || s == o->tensors.end() || g == o->tensors.end()) return B200_EINVAL;
    if (p->second.dtype != "U8" || s->second.dtype != "F8_E4M3" || g->second.dtype != "F32" || p->second.shape.size() != 2 ||
        s->second.shape.size() != 2 || g->second.bytes != 4) return B200_ESHAPE;
    const long N = p->second.shape[0], K = p->second.shape[1] * 2;
    if (s->second.shape[0] != N || s->second.shape[1] * 16 != K || p->second.bytes != (size_t)(N * K / 2) || s->second.bytes != (size_t)(N * K / 16)) return B200_ESHAPE;
    out->packed = p->second.data; out->scale = s->second.data;
    memcpy(&out->gscale, g->second.data, 4);
    out->N = (int)N; out->K = (int)K;
    return B200_OK;
}
