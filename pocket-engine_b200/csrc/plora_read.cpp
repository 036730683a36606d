// Adapter files into the registry's host image: PEFT directories (adapter_config.json +
// *.safetensors; src/lora.rs:148-233, src/source.rs:28-186) and llama.cpp GGUF adapters
// (src/lora.rs:237-281, src/source.rs:477-551), then Prep::read's dispatch (src/lora.rs:298-306).
// Plain host code: callable from any thread, no CUDA calls of its own (plora_adapter_prepare pins the
// slab when the handle has a device).
#include <dirent.h>
#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "plora_internal.h"

void plora_set_adapter_error(const std::string& text);  // plora_host.cpp: the thread-local text of plora_adapter_error

namespace {

struct Fail {
    std::string text;
};
[[noreturn]] void fail(const std::string& t) { throw Fail{t}; }

// ------------------------------------------------------------------ a small JSON reader

struct JVal {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double n = 0;
    std::string s;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal* get(const std::string& k) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj)
            if (kv.first == k) return &kv.second;
        return nullptr;
    }
};

struct JParser {
    const char* p;
    const char* end;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
    }
    [[noreturn]] void bad(const char* what) { fail(std::string("JSON: ") + what + " at byte " + std::to_string(p - start)); }
    const char* start;
    JVal value(int depth = 0) {
        if (depth > 64) bad("nesting too deep");
        ws();
        if (p >= end) bad("unexpected end");
        JVal v;
        switch (*p) {
            case '{': {
                v.kind = JVal::Obj;
                p++;
                ws();
                if (p < end && *p == '}') {
                    p++;
                    return v;
                }
                for (;;) {
                    ws();
                    if (p >= end || *p != '"') bad("expected a key");
                    std::string k = str();
                    ws();
                    if (p >= end || *p != ':') bad("expected ':'");
                    p++;
                    v.obj.emplace_back(std::move(k), value(depth + 1));
                    ws();
                    if (p < end && *p == ',') {
                        p++;
                        continue;
                    }
                    if (p < end && *p == '}') {
                        p++;
                        return v;
                    }
                    bad("expected ',' or '}'");
                }
            }
            case '[': {
                v.kind = JVal::Arr;
                p++;
                ws();
                if (p < end && *p == ']') {
                    p++;
                    return v;
                }
                for (;;) {
                    v.arr.push_back(value(depth + 1));
                    ws();
                    if (p < end && *p == ',') {
                        p++;
                        continue;
                    }
                    if (p < end && *p == ']') {
                        p++;
                        return v;
                    }
                    bad("expected ',' or ']'");
                }
            }
            case '"':
                v.kind = JVal::Str;
                v.s = str();
                return v;
            case 't':
                lit("true");
                v.kind = JVal::Bool;
                v.b = true;
                return v;
            case 'f':
                lit("false");
                v.kind = JVal::Bool;
                return v;
            case 'n':
                lit("null");
                return v;
            default: {
                char* e = nullptr;
                std::string tok;
                const char* q = p;
                while (q < end && (std::strchr("+-.eE", *q) || (*q >= '0' && *q <= '9'))) q++;
                tok.assign(p, q);
                if (tok.empty()) bad("unexpected character");
                v.n = std::strtod(tok.c_str(), &e);
                if (*e) bad("malformed number");
                v.kind = JVal::Num;
                p = q;
                return v;
            }
        }
    }
    void lit(const char* w) {
        const size_t n = std::strlen(w);
        if ((size_t)(end - p) < n || std::memcmp(p, w, n) != 0) bad("unexpected literal");
        p += n;
    }
    std::string str() {
        std::string out;
        p++;  // opening quote
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) bad("unfinished escape");
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (end - p < 5) bad("unfinished \\u escape");
                        unsigned cp = (unsigned)std::strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
                        p += 4;
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) {
                            out += (char)(0xC0 | (cp >> 6));
                            out += (char)(0x80 | (cp & 0x3F));
                        } else {
                            out += (char)(0xE0 | (cp >> 12));
                            out += (char)(0x80 | ((cp >> 6) & 0x3F));
                            out += (char)(0x80 | (cp & 0x3F));
                        }
                        break;
                    }
                    default: out += *p;  // \" \\ \/
                }
                p++;
            } else {
                out += *p++;
            }
        }
        if (p >= end) bad("unfinished string");
        p++;
        return out;
    }
};

JVal parse_json(const std::string& text) {
    JParser ps{text.data(), text.data() + text.size(), text.data()};
    JVal v = ps.value();
    ps.ws();
    if (ps.p != ps.end) ps.bad("trailing characters");
    return v;
}

std::string read_file(const std::string& path, const std::string& label) {
    std::ifstream f(path, std::ios::binary);
    if (!f) fail(label + ": " + std::strerror(errno));
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

// ------------------------------------------------------------------ number formats

float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {  // subnormal: renormalise
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// ------------------------------------------------------------------ safetensors (src/source.rs:28-186)

struct StEntry {
    size_t file = 0;
    std::string dtype;
    std::vector<size_t> shape;
    uint64_t start = 0, end = 0;  // byte range in the file
};

struct Checkpoint {
    std::vector<std::string> paths;
    std::vector<uint64_t> sizes;
    std::map<std::string, StEntry> index;  // sorted by name, as Checkpoint::names returns them

    explicit Checkpoint(const std::string& dir) {
        std::vector<std::string> names;
        DIR* d = opendir(dir.c_str());
        if (!d) fail(dir + ": " + std::strerror(errno));
        while (dirent* e = readdir(d)) {
            std::string n = e->d_name;
            if (n.size() > 12 && n.compare(n.size() - 12, 12, ".safetensors") == 0) names.push_back(n);
        }
        closedir(d);
        std::sort(names.begin(), names.end());
        if (names.empty()) fail("no safetensors in " + dir);
        for (size_t i = 0; i < names.size(); i++) {
            const std::string path = dir + "/" + names[i];
            std::ifstream f(path, std::ios::binary);
            if (!f) fail(path + ": " + std::strerror(errno));
            f.seekg(0, std::ios::end);
            const uint64_t size = (uint64_t)f.tellg();
            f.seekg(0);
            uint64_t n = 0;
            if (size < 8 || !f.read(reinterpret_cast<char*>(&n), 8) || n > size - 8) fail(path + ": not a safetensors file");
            std::string header((size_t)n, '\0');
            if (!f.read(&header[0], (std::streamsize)n)) fail(path + ": truncated header");
            JVal meta;
            try {
                meta = parse_json(header);
            } catch (const Fail& e) {
                fail(path + ": " + e.text);
            }
            if (meta.kind != JVal::Obj) fail(path + ": header is not an object");
            for (auto& kv : meta.obj) {
                if (kv.first == "__metadata__") continue;
                const JVal *dt = kv.second.get("dtype"), *sh = kv.second.get("shape"), *off = kv.second.get("data_offsets");
                if (!dt || dt->kind != JVal::Str || !sh || sh->kind != JVal::Arr || !off || off->kind != JVal::Arr ||
                    off->arr.size() != 2)
                    fail(path + ": malformed entry for " + kv.first);
                StEntry e;
                e.file = i;
                e.dtype = dt->s;
                for (auto& x : sh->arr) e.shape.push_back((size_t)x.n);
                e.start = 8 + n + (uint64_t)off->arr[0].n;
                e.end = 8 + n + (uint64_t)off->arr[1].n;
                index[kv.first] = e;
            }
            paths.push_back(path);
            sizes.push_back(size);
        }
    }

    const std::vector<size_t>& shape(const std::string& full) const {
        auto it = index.find(full);
        if (it == index.end()) fail("missing tensor " + full);
        return it->second.shape;
    }

    // a tensor as f32, by its full name (src/source.rs:160-186)
    std::vector<float> f32_full(const std::string& full, size_t numel) const {
        auto it = index.find(full);
        if (it == index.end()) fail("missing tensor " + full);
        const StEntry& e = it->second;
        if (e.end < e.start || e.end > sizes[e.file]) fail(full + " runs past the end of its file");
        size_t n = 1;
        for (size_t d : e.shape) n *= d;
        if (n != numel) fail(full + ": shape does not hold " + std::to_string(numel) + " elements");
        const size_t es = e.dtype == "F32" ? 4 : e.dtype == "BF16" ? 2 : 0;
        if (!es) fail(full + ": unsupported dtype " + e.dtype);
        if ((e.end - e.start) != (uint64_t)numel * es) fail(full + ": byte range does not match its shape");
        std::vector<unsigned char> raw((size_t)(e.end - e.start));
        std::ifstream f(paths[e.file], std::ios::binary);
        f.seekg((std::streamoff)e.start);
        if (!f.read(reinterpret_cast<char*>(raw.data()), (std::streamsize)raw.size())) fail(full + ": read failed");
        std::vector<float> out(numel);
        if (es == 4) {
            std::memcpy(out.data(), raw.data(), numel * 4);
        } else {
            for (size_t i = 0; i < numel; i++) {
                uint16_t h;
                std::memcpy(&h, raw.data() + 2 * i, 2);
                out[i] = bf16_to_f32(h);
            }
        }
        return out;
    }
};

// ------------------------------------------------------------------ modules

struct Module {  // src/lora.rs:91-95 keyed by (layer, module path)
    int layer = 0, r = 0;
    std::string module;
    std::vector<float> a, b;
};

bool ends_with(const std::string& s, const std::string& suffix) {
    return s.size() >= suffix.size() && s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
}

// src/lora.rs:148-233
std::vector<Module> read_peft(const std::string& dir) {
    const std::string cfg_path = dir + "/adapter_config.json";
    JVal cfg;
    const std::string text = read_file(cfg_path, cfg_path);
    try {
        cfg = parse_json(text);
    } catch (const Fail& e) {
        fail("adapter_config.json: " + e.text);
    }
    auto flag = [&](const char* k) {
        const JVal* v = cfg.get(k);
        return v && v->kind == JVal::Bool && v->b;
    };
    if (flag("use_dora")) fail("DoRA adapters are not supported");
    if (const JVal* v = cfg.get("modules_to_save"))
        if (v->kind != JVal::Null && (v->kind != JVal::Arr || !v->arr.empty()))
            fail("adapters with modules_to_save (full embedding or output layers) are not supported");
    if (const JVal* v = cfg.get("bias"))
        if (v->kind == JVal::Str && v->s != "none") fail("adapters with trained biases are not supported");
    if (const JVal* v = cfg.get("alpha_pattern"))
        if (v->kind == JVal::Obj && !v->obj.empty()) fail("adapters with alpha_pattern are not supported");
    double alpha = 8.0;
    if (const JVal* v = cfg.get("lora_alpha"))
        if (v->kind == JVal::Num) alpha = v->n;
    const bool rslora = flag("use_rslora");
    Checkpoint ck(dir);
    std::vector<Module> out;
    for (auto& kv : ck.index) {
        const std::string& name = kv.first;
        if (!ends_with(name, ".lora_A.weight")) continue;
        const std::string stem = name.substr(0, name.size() - 14);
        if (stem.find("visual") != std::string::npos) fail("adapters for the vision encoder are not supported");
        if (stem.find(".mtp.") != std::string::npos) continue;
        const size_t at = stem.rfind("layers.");
        if (at == std::string::npos) fail(name + ": not a decoder layer");
        const std::string rest = stem.substr(at + 7);
        const size_t dot = rest.find('.');
        if (dot == std::string::npos || dot == 0) fail(name + ": unexpected name");
        const std::string layer_s = rest.substr(0, dot);
        if (layer_s.find_first_not_of("0123456789") != std::string::npos || layer_s.size() > 9) fail(name + ": unexpected name");
        const std::vector<size_t>& ashape = ck.shape(name);
        const std::vector<size_t>& bshape = ck.shape(stem + ".lora_B.weight");
        if (ashape.size() != 2 || bshape.size() != 2) fail(stem + ": LoRA factors must be matrices");
        const size_t r = ashape[0], cols = ashape[1], rows = bshape[0];
        if (bshape[1] != r)
            fail(stem + ": A is rank " + std::to_string(r) + ", B [" + std::to_string(bshape[0]) + ", " +
                 std::to_string(bshape[1]) + "]");
        const float scale = (float)(alpha / (rslora ? std::sqrt((double)r) : (double)r));
        Module m;
        m.layer = std::atoi(layer_s.c_str());
        m.module = rest.substr(dot + 1);
        m.r = (int)r;
        m.a = ck.f32_full(name, r * cols);
        m.b = ck.f32_full(stem + ".lora_B.weight", rows * r);
        for (float& x : m.b) x *= scale;  // in f32, before any bf16 rounding (:225-228)
        out.push_back(std::move(m));
    }
    return out;
}

// ------------------------------------------------------------------ GGUF (the published llama.cpp container format)

struct GgufTensor {
    std::vector<uint64_t> dims;  // innermost first
    uint32_t type = 0;
    uint64_t offset = 0;  // from the start of the data section
};

struct Gguf {
    std::string path;
    std::map<std::string, JVal> kv;  // scalars and strings only; arrays are skipped
    std::map<std::string, GgufTensor> tensors;
    uint64_t data_start = 0, size = 0;

    struct Cursor {
        const unsigned char* p;
        const unsigned char* end;
        const std::string* path;
        template <typename T>
        T get() {
            if ((size_t)(end - p) < sizeof(T)) fail(*path + ": truncated GGUF header");
            T v;
            std::memcpy(&v, p, sizeof(T));
            p += sizeof(T);
            return v;
        }
        std::string str() {
            const uint64_t n = get<uint64_t>();
            if ((uint64_t)(end - p) < n) fail(*path + ": truncated GGUF string");
            std::string s(reinterpret_cast<const char*>(p), (size_t)n);
            p += n;
            return s;
        }
    };

    static size_t scalar_size(uint32_t t) {
        switch (t) {
            case 0: case 1: case 7: return 1;
            case 2: case 3: return 2;
            case 4: case 5: case 6: return 4;
            case 10: case 11: case 12: return 8;
            default: return 0;
        }
    }

    JVal value(Cursor& c, uint32_t t, bool keep) {
        JVal v;
        switch (t) {
            case 0: v.kind = JVal::Num; v.n = c.get<uint8_t>(); break;
            case 1: v.kind = JVal::Num; v.n = c.get<int8_t>(); break;
            case 2: v.kind = JVal::Num; v.n = c.get<uint16_t>(); break;
            case 3: v.kind = JVal::Num; v.n = c.get<int16_t>(); break;
            case 4: v.kind = JVal::Num; v.n = c.get<uint32_t>(); break;
            case 5: v.kind = JVal::Num; v.n = c.get<int32_t>(); break;
            case 6: v.kind = JVal::Num; v.n = c.get<float>(); break;
            case 7: v.kind = JVal::Bool; v.b = c.get<uint8_t>() != 0; break;
            case 8: v.kind = JVal::Str; v.s = c.str(); break;
            case 10: v.kind = JVal::Num; v.n = (double)c.get<uint64_t>(); break;
            case 11: v.kind = JVal::Num; v.n = (double)c.get<int64_t>(); break;
            case 12: v.kind = JVal::Num; v.n = c.get<double>(); break;
            case 9: {
                const uint32_t et = c.get<uint32_t>();
                const uint64_t n = c.get<uint64_t>();
                if (et == 8) {
                    for (uint64_t i = 0; i < n; i++) c.str();
                } else if (et == 9) {
                    for (uint64_t i = 0; i < n; i++) value(c, 9, false);
                } else {
                    const size_t es = scalar_size(et);
                    if (!es || (uint64_t)(c.end - c.p) / es < n) fail(path + ": malformed GGUF array");
                    c.p += n * es;
                }
                v.kind = JVal::Arr;
                break;
            }
            default: fail(path + ": unknown GGUF value type " + std::to_string(t));
        }
        (void)keep;
        return v;
    }

    explicit Gguf(const std::string& file) : path(file) {
        const std::string raw = read_file(file, file);
        size = raw.size();
        Cursor c{reinterpret_cast<const unsigned char*>(raw.data()), reinterpret_cast<const unsigned char*>(raw.data()) + raw.size(),
                 &path};
        if (raw.size() < 24 || std::memcmp(raw.data(), "GGUF", 4) != 0) fail(file + " is not a GGUF file");
        c.p += 4;
        const uint32_t version = c.get<uint32_t>();
        if (version < 2 || version > 3) fail(file + ": unsupported GGUF version " + std::to_string(version));
        const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
        for (uint64_t i = 0; i < n_kv; i++) {
            std::string key = c.str();
            const uint32_t t = c.get<uint32_t>();
            kv[key] = value(c, t, true);
        }
        for (uint64_t i = 0; i < n_tensors; i++) {
            std::string name = c.str();
            GgufTensor t;
            const uint32_t nd = c.get<uint32_t>();
            if (nd > 4) fail(file + ": tensor " + name + " has " + std::to_string(nd) + " dimensions");
            for (uint32_t d = 0; d < nd; d++) t.dims.push_back(c.get<uint64_t>());
            t.type = c.get<uint32_t>();
            t.offset = c.get<uint64_t>();
            tensors[name] = t;
        }
        uint64_t align = 32;
        auto it = kv.find("general.alignment");
        if (it != kv.end() && it->second.kind == JVal::Num && it->second.n >= 1) align = (uint64_t)it->second.n;
        const uint64_t at = (uint64_t)(c.p - reinterpret_cast<const unsigned char*>(raw.data()));
        data_start = (at + align - 1) / align * align;
        data_ = raw;  // adapters are small: keep the file in memory
    }

    // F32 (0), F16 (1) or BF16 (30) to f32 (src/source.rs:529-551)
    std::vector<float> f32(const std::string& base, const GgufTensor& t) const {
        size_t n = 1;
        for (uint64_t d : t.dims) n *= (size_t)d;
        const size_t es = t.type == 0 ? 4 : (t.type == 1 || t.type == 30) ? 2 : 0;
        if (!es) fail(base + ": LoRA tensors must be F32, F16 or BF16");
        const uint64_t at = data_start + t.offset;
        if (at > size || (size - at) / es < n) fail(base + " runs past the end of its file");
        const unsigned char* p = reinterpret_cast<const unsigned char*>(data_.data()) + at;
        std::vector<float> out(n);
        if (es == 4) {
            std::memcpy(out.data(), p, n * 4);
        } else {
            for (size_t i = 0; i < n; i++) {
                uint16_t h;
                std::memcpy(&h, p + 2 * i, 2);
                out[i] = t.type == 1 ? f16_to_f32(h) : bf16_to_f32(h);
            }
        }
        return out;
    }

   private:
    std::string data_;
};

// src/source.rs:499-526, the decoder-layer names
std::string gguf_layer_name(int layer, const std::string& module) {
    static const std::pair<const char*, const char*> map[] = {
        {"mlp.gate_proj", "ffn_gate"},          {"mlp.up_proj", "ffn_up"},
        {"mlp.down_proj", "ffn_down"},          {"self_attn.q_proj", "attn_q"},
        {"self_attn.k_proj", "attn_k"},         {"self_attn.v_proj", "attn_v"},
        {"self_attn.o_proj", "attn_output"},    {"linear_attn.in_proj_qkv", "attn_qkv"},
        {"linear_attn.in_proj_z", "attn_gate"}, {"linear_attn.in_proj_b", "ssm_beta"},
        {"linear_attn.in_proj_a", "ssm_alpha"}, {"linear_attn.out_proj", "ssm_out"},
    };
    std::string mapped = module;
    for (auto& m : map)
        if (module == m.first) mapped = m.second;
    return "blk." + std::to_string(layer) + "." + mapped + ".weight";
}

// src/lora.rs:237-281
std::vector<Module> read_gguf(const std::string& path, const std::vector<SiteInfo>& sites) {
    Gguf g(path);
    auto ty = g.kv.find("general.type");
    if (ty == g.kv.end() || ty->second.kind != JVal::Str || ty->second.s != "adapter") fail(path + " is not a LoRA adapter");
    bool has_alpha = false;
    double alpha = 0;
    auto al = g.kv.find("adapter.lora.alpha");
    if (al != g.kv.end() && al->second.kind == JVal::Num) {
        has_alpha = true;
        alpha = al->second.n;
    }
    std::vector<Module> out;
    for (auto& site : sites) {
        for (auto& part : site.parts) {
            const std::string base = gguf_layer_name(site.layer, part.module);
            auto ta = g.tensors.find(base + ".lora_a"), tb = g.tensors.find(base + ".lora_b");
            if (ta == g.tensors.end() || tb == g.tensors.end()) continue;
            if (ta->second.dims.size() != 2 || tb->second.dims.size() != 2) fail(base + ": unexpected LoRA shapes");
            // the innermost dimension comes first: A is (cols, r), B (r, rows)
            const uint64_t cols = ta->second.dims[0], r = ta->second.dims[1], rows = tb->second.dims[1];
            if (tb->second.dims[0] != r || cols != (uint64_t)site.cols || rows != (uint64_t)part.rows)
                fail(base + ": unexpected LoRA shapes");
            Module m;
            m.layer = site.layer;
            m.module = part.module;
            m.r = (int)r;
            m.a = g.f32(base, ta->second);
            m.b = g.f32(base, tb->second);
            const float scale = has_alpha ? (float)(alpha / (double)r) : 1.0f;
            for (float& x : m.b) x *= scale;
            out.push_back(std::move(m));
        }
    }
    if (out.empty()) fail(path + ": no LoRA tensors for this model");
    return out;
}

}  // namespace

// Prep::read (src/lora.rs:298-306): a PEFT directory or a GGUF file, laid out as its GPU slot will hold it.
extern "C" int plora_adapter_read(const plora_t* h, const char* name, const char* path, plora_adapter_t** out) {
    if (!h || !name || !path || !out) return PLORA_ERR_ARG;
    *out = nullptr;
    try {
        struct stat st;
        if (stat(path, &st) != 0) fail(std::string(path) + ": " + std::strerror(errno));
        const bool dir = S_ISDIR(st.st_mode);
        std::vector<Module> mods = dir ? read_peft(path) : read_gguf(path, h->sites);
        std::vector<plora_module> view(mods.size());
        for (size_t i = 0; i < mods.size(); i++) {
            view[i].layer = mods[i].layer;
            view[i].r = mods[i].r;
            view[i].module = mods[i].module.c_str();
            view[i].a = mods[i].a.data();
            view[i].b = mods[i].b.data();
            view[i].a_len = mods[i].a.size();
            view[i].b_len = mods[i].b.size();
        }
        // PEFT files hold the grouped value-head order, llama.cpp adapters the tiled one (:232, :280)
        return plora_adapter_prepare(h, name, view.data(), (int)view.size(), dir ? 0 : 1, out);
    } catch (const Fail& e) {
        plora_set_adapter_error(e.text);
        return PLORA_ERR_CONFIG;
    } catch (const std::bad_alloc&) {
        plora_set_adapter_error("out of memory reading the adapter");
        return PLORA_ERR_CONFIG;
    }
}
