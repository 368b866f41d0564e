// Reader of a `.gturbo` model directory and its upload into HBM.
//
// A directory holds
//   manifest.json                      dimensions, quantisation slots, file table
//   packed_experts/layout.json         per layer: file name and, per expert, blob offset and sub-tensor table
//   packed_experts/<layer file>        experts_per_layer blobs of expert_stride bytes
//   model_weights.bin                  [24-byte header | 72-byte entries | names | padding] + resident tensors
//
// This file restates the format rules of the reference's readers
//   Sources/TurboFieldfareFormat/GTurboFormatV1.swift:3-23             constants, dtype codes
//   Sources/TurboFieldfareFormat/GTurboManifestV1.swift:172-268        manifest validation
//   Sources/TurboFieldfareFormat/GTurboPackedExpertsLayoutV1.swift:86-211   layout validation, cross-check
//   Sources/TurboFieldfareFormat/GTurboResidentIndexV1.swift:40-158    resident index decoding
//   Sources/TurboFieldfare/Infrastructure/ModelIO/ManifestReader.swift:89-152
//   Sources/TurboFieldfare/Infrastructure/ModelIO/PackedExpertsLayout.swift:82-119
//   Sources/TurboFieldfare/Runtime/Inference/Model.swift:195-233       name -> payload-relative tensor view
//   Sources/TurboFieldfare/Runtime/Inference/ModelExpertIO.swift:21-40 nine routed-expert offsets
//   Sources/TurboFieldfare/Runtime/Inference/RealForwardRunner.swift:352-376   1/sqrt(D) folded into router.scale
// and replaces the SSD streamer with one upload of every blob into the expert pool.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "turbofieldfare_cuda.h"

namespace tf {
void set_global_error(const char* fmt, ...);
}

namespace {

constexpr uint64_t kAlignment = 16384;             // GTurboFormatV1.alignmentBytes
constexpr uint64_t kHeaderBytes = 24;              // residentHeaderBytes
constexpr uint64_t kEntryBytes = 72;               // residentEntryBytes
constexpr uint64_t kIndexMaxBytes = 16u << 20;     // residentIndexMaxBytes
constexpr uint64_t kManifestMaxBytes = 4u << 20;   // ManifestReader.defaultMaxBytes
constexpr uint64_t kLayoutMaxBytes = 16u << 20;    // PackedExpertsLayoutReader.defaultMaxBytes

struct FormatError {
    tf_status code;
    std::string text;
};

[[noreturn]] void raise(tf_status code, const char* fmt, ...) {
    char buf[768];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    throw FormatError{code, buf};
}

uint64_t checked_add(uint64_t a, uint64_t b, const char* field) {
    uint64_t r;
    if (__builtin_add_overflow(a, b, &r)) raise(TF_ERR_FORMAT_OVERFLOW, "%s: arithmetic overflow", field);
    return r;
}
uint64_t checked_mul(uint64_t a, uint64_t b, const char* field) {
    uint64_t r;
    if (__builtin_mul_overflow(a, b, &r)) raise(TF_ERR_FORMAT_OVERFLOW, "%s: arithmetic overflow", field);
    return r;
}

// ---------------------------------------------------------------------------
// A small JSON reader (objects keep their members in document order)
// ---------------------------------------------------------------------------
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    bool is_uint = false;        // the literal was a non-negative integer that fits 64 bits
    uint64_t u = 0;
    bool is_int = false;         // the literal was an integer (possibly negative) that fits int64
    int64_t i = 0;
    std::string str;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* find(const std::string& key) const {
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
};

class JsonParser {
public:
    JsonParser(const char* p, size_t n, const char* doc) : p_(p), end_(p + n), doc_(doc) {}
    Json parse() {
        Json v = value(0);
        skip_ws();
        if (p_ != end_) bad("trailing characters after the document");
        return v;
    }

private:
    const char* p_;
    const char* end_;
    const char* doc_;

    [[noreturn]] void bad(const char* what) { raise(TF_ERR_FORMAT_INVALID, "%s: %s", doc_, what); }
    void skip_ws() {
        while (p_ != end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\r' || *p_ == '\t')) ++p_;
    }
    bool eat(const char* word) {
        const size_t n = strlen(word);
        if ((size_t)(end_ - p_) >= n && memcmp(p_, word, n) == 0) { p_ += n; return true; }
        return false;
    }
    static void append_utf8(std::string& s, uint32_t cp) {
        if (cp < 0x80) s += (char)cp;
        else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
        else { s += (char)(0xF0 | (cp >> 18)); s += (char)(0x80 | ((cp >> 12) & 0x3F)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
    }
    uint32_t hex4() {
        if (end_ - p_ < 4) bad("truncated \\u escape");
        uint32_t v = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= (uint32_t)(c - '0');
            else if (c >= 'a' && c <= 'f') v |= (uint32_t)(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= (uint32_t)(c - 'A' + 10);
            else bad("bad \\u escape");
        }
        return v;
    }
    std::string string_body() {
        std::string s;
        ++p_;   // opening quote
        for (;;) {
            if (p_ == end_) bad("unterminated string");
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') return s;
            if (c < 0x20) bad("control character in string");
            if (c != '\\') { s += (char)c; continue; }
            if (p_ == end_) bad("unterminated escape");
            const char e = *p_++;
            switch (e) {
                case '"': s += '"'; break;
                case '\\': s += '\\'; break;
                case '/': s += '/'; break;
                case 'b': s += '\b'; break;
                case 'f': s += '\f'; break;
                case 'n': s += '\n'; break;
                case 'r': s += '\r'; break;
                case 't': s += '\t'; break;
                case 'u': {
                    uint32_t cp = hex4();
                    if (cp >= 0xD800 && cp <= 0xDBFF) {
                        if (!(end_ - p_ >= 2 && p_[0] == '\\' && p_[1] == 'u')) bad("lone surrogate");
                        p_ += 2;
                        const uint32_t lo = hex4();
                        if (lo < 0xDC00 || lo > 0xDFFF) bad("bad surrogate pair");
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
                        bad("lone surrogate");
                    }
                    append_utf8(s, cp);
                    break;
                }
                default: bad("unknown escape");
            }
        }
    }
    Json number() {
        const char* start = p_;
        if (p_ != end_ && *p_ == '-') ++p_;
        if (p_ == end_ || *p_ < '0' || *p_ > '9') bad("malformed number");
        if (*p_ == '0') ++p_;
        else while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        bool integral = true;
        if (p_ != end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9') bad("malformed fraction");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ != end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ != end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ == end_ || *p_ < '0' || *p_ > '9') bad("malformed exponent");
            while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        Json v;
        v.kind = Json::Number;
        const std::string text(start, p_);
        v.num = strtod(text.c_str(), nullptr);
        if (integral) {
            errno = 0;
            if (text[0] != '-') {
                const unsigned long long u = strtoull(text.c_str(), nullptr, 10);
                if (errno == 0) { v.is_uint = true; v.u = u; if (u <= (unsigned long long)INT64_MAX) { v.is_int = true; v.i = (int64_t)u; } }
            } else {
                const long long i = strtoll(text.c_str(), nullptr, 10);
                if (errno == 0) { v.is_int = true; v.i = i; }
            }
        }
        return v;
    }
    Json value(int depth) {
        if (depth > 64) bad("nesting too deep");
        skip_ws();
        if (p_ == end_) bad("unexpected end of document");
        Json v;
        const char c = *p_;
        if (c == '{') {
            ++p_;
            v.kind = Json::Object;
            skip_ws();
            if (p_ != end_ && *p_ == '}') { ++p_; return v; }
            for (;;) {
                skip_ws();
                if (p_ == end_ || *p_ != '"') bad("expected a member name");
                std::string key = string_body();
                skip_ws();
                if (p_ == end_ || *p_ != ':') bad("expected ':'");
                ++p_;
                Json member = value(depth + 1);
                if (v.find(key)) bad("duplicate member name");
                v.members.emplace_back(std::move(key), std::move(member));
                skip_ws();
                if (p_ == end_) bad("unterminated object");
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == '}') { ++p_; return v; }
                bad("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p_;
            v.kind = Json::Array;
            skip_ws();
            if (p_ != end_ && *p_ == ']') { ++p_; return v; }
            for (;;) {
                v.items.push_back(value(depth + 1));
                skip_ws();
                if (p_ == end_) bad("unterminated array");
                if (*p_ == ',') { ++p_; continue; }
                if (*p_ == ']') { ++p_; return v; }
                bad("expected ',' or ']'");
            }
        }
        if (c == '"') { v.kind = Json::String; v.str = string_body(); return v; }
        if (eat("true")) { v.kind = Json::Bool; v.b = true; return v; }
        if (eat("false")) { v.kind = Json::Bool; v.b = false; return v; }
        if (eat("null")) { v.kind = Json::Null; return v; }
        return number();
    }
};

// typed member access: a missing or mistyped member is what JSONDecoder would reject
const Json& need(const Json& obj, const char* key, Json::Kind kind, const char* doc) {
    if (obj.kind != Json::Object) raise(TF_ERR_FORMAT_INVALID, "%s: expected an object around \"%s\"", doc, key);
    const Json* v = obj.find(key);
    if (!v) raise(TF_ERR_FORMAT_INVALID, "%s: member \"%s\" is missing", doc, key);
    if (v->kind != kind) raise(TF_ERR_FORMAT_INVALID, "%s: member \"%s\" has the wrong type", doc, key);
    return *v;
}
uint64_t need_u64(const Json& obj, const char* key, const char* doc) {
    const Json& v = need(obj, key, Json::Number, doc);
    if (!v.is_uint) raise(TF_ERR_FORMAT_INVALID, "%s: member \"%s\" is not an unsigned integer", doc, key);
    return v.u;
}
int64_t need_int(const Json& obj, const char* key, const char* doc) {
    const Json& v = need(obj, key, Json::Number, doc);
    if (!v.is_int) raise(TF_ERR_FORMAT_INVALID, "%s: member \"%s\" is not an integer", doc, key);
    return v.i;
}
bool optional_int(const Json& obj, const char* key, const char* doc, int64_t* out) {
    const Json* v = obj.kind == Json::Object ? obj.find(key) : nullptr;
    if (!v || v->kind == Json::Null) return false;
    if (v->kind != Json::Number || !v->is_int) raise(TF_ERR_FORMAT_INVALID, "%s: member \"%s\" is not an integer", doc, key);
    *out = v->i;
    return true;
}

// ---------------------------------------------------------------------------
// Paths (GTurboFormatV1.swift:52-77)
// ---------------------------------------------------------------------------
std::vector<std::string> split_path(const std::string& path) {
    std::vector<std::string> parts;
    size_t start = 0;
    for (;;) {
        const size_t slash = path.find('/', start);
        parts.push_back(path.substr(start, slash == std::string::npos ? std::string::npos : slash - start));
        if (slash == std::string::npos) break;
        start = slash + 1;
    }
    return parts;
}
void validate_relative_path(const std::string& path, const char* field) {
    if (path.empty() || path[0] == '/' || path.find('\0') != std::string::npos)
        raise(TF_ERR_FORMAT_INVALID, "%s: unsafe relative path", field);
    for (const std::string& part : split_path(path))
        if (part.empty() || part == "." || part == "..") raise(TF_ERR_FORMAT_INVALID, "%s: non-canonical path", field);
}
void validate_basename(const std::string& name, const char* field) {
    validate_relative_path(name, field);
    if (name.find('/') != std::string::npos) raise(TF_ERR_FORMAT_INVALID, "%s: expected basename", field);
}
// Case-insensitive key of a file name. The reference also applies Unicode canonical composition; names
// outside ASCII are compared byte for byte here.
std::string filesystem_key(const std::string& path) {
    std::string k = path;
    for (char& c : k)
        if (c >= 'A' && c <= 'Z') c = (char)(c - 'A' + 'a');
    return k;
}

// ---------------------------------------------------------------------------
// Parsed documents
// ---------------------------------------------------------------------------
struct SubTensor {
    uint64_t offset = 0, size = 0;
    std::string dtype;
    std::vector<uint32_t> shape;
    int bits = 0;          // 0: absent
};
struct Expert {
    int logical = 0, physical = 0;
    uint64_t offset = 0, size = 0;
    std::map<std::string, SubTensor> tensors;
};
struct Layer {
    int layer = 0;
    std::string file;
    std::vector<Expert> experts;     // sorted by logical id
};
struct Layout {
    uint64_t expert_stride = 0;
    int num_layers = 0, experts_per_layer = 0;
    std::vector<Layer> layers;       // sorted by layer id
};
struct QuantSlot {
    int weight_bits = 0, group_size = 0;
    std::string scheme, scale_type, bias_type;
};
struct Manifest {
    int version_major = 0, version_minor = 0;
    std::string model_id;
    int hidden = 0, ffn = 0, moe_ffn = 0, num_layers = 0, num_experts = 0, top_k = 0, vocab = 0;
    std::string activation;
    bool has_quant = false;
    QuantSlot q_embedding, q_attention, q_router, q_shared, q_routed;
    std::map<std::string, uint64_t> file_sizes;
    std::map<std::string, std::string> file_sha256;
    int experts_per_layer = 0, layers = 0;
    uint64_t expert_stride = 0;
};
struct ResidentEntry {
    std::string name;
    uint8_t dtype = 0;
    uint64_t file_offset = 0, size = 0, scale_offset = 0, scale_size = 0, bias_offset = 0, bias_size = 0;
    uint32_t shape[4] = {0, 0, 0, 0};
};
struct ResidentIndex {
    uint64_t index_size = 0, resident_size = 0, entry_count = 0;
    std::vector<ResidentEntry> entries;
    std::map<std::string, size_t> by_name;
};

std::string lower(std::string s) {
    for (char& c : s)
        if (c >= 'A' && c <= 'Z') c = (char)(c - 'A' + 'a');
    return s;
}

QuantSlot parse_slot(const Json& quant, const char* key) {
    const char* doc = "manifest.json";
    const Json& s = need(quant, key, Json::Object, doc);
    QuantSlot q;
    q.weight_bits = (int)need_int(s, "weightBits", doc);
    q.group_size = (int)need_int(s, "groupSize", doc);
    q.scheme = need(s, "scheme", Json::String, doc).str;
    q.scale_type = need(s, "scaleType", Json::String, doc).str;
    q.bias_type = need(s, "biasType", Json::String, doc).str;
    // GTurboManifestV1.swift:216-230 and ManifestReader.swift:135-152
    if (q.weight_bits <= 0 || q.weight_bits > 32 || q.group_size <= 0)
        raise(TF_ERR_FORMAT_INVALID, "manifest.quant.%s: invalid quantization slot", key);
    if (lower(q.scheme) != "affine" || lower(q.scale_type) != "bf16" || lower(q.bias_type) != "bf16" ||
        q.group_size != TF_GROUP_SIZE)
        raise(TF_ERR_FORMAT_INVALID, "unsupported quantization for %s", key);
    return q;
}

Manifest parse_manifest(const char* bytes, size_t n) {
    const char* doc = "manifest.json";
    const Json root = JsonParser(bytes, n, doc).parse();
    Manifest m;
    if (need(root, "magic", Json::String, doc).str != "GTURBO") raise(TF_ERR_FORMAT_INVALID, "manifest.magic: expected GTURBO");
    m.version_major = (int)need_int(root, "versionMajor", doc);
    m.version_minor = (int)need_int(root, "versionMinor", doc);
    if (m.version_major != 1 || m.version_minor < 0)
        raise(TF_ERR_UNSUPPORTED, "manifest.version: unsupported version %d.%d", m.version_major, m.version_minor);
    const Json& flags = need(root, "flags", Json::Object, doc);
    for (const auto& f : flags.members) {
        if (f.first != "streamingPresent" && f.first != "turboQuantKV" && f.first != "aneSharedExpert")
            raise(TF_ERR_FORMAT_INVALID, "manifest.flags.%s: unknown v1 flag", f.first.c_str());
        if (f.second.kind != Json::Bool) raise(TF_ERR_FORMAT_INVALID, "manifest.flags.%s: not a boolean", f.first.c_str());
        if (f.first == "turboQuantKV" && f.second.b)
            raise(TF_ERR_FORMAT_INVALID, "manifest requests removed TurboQuant KV runtime support");
    }
    m.model_id = need(root, "modelID", Json::String, doc).str;
    m.experts_per_layer = (int)need_int(root, "expertsPerLayer", doc);
    m.layers = (int)need_int(root, "numLayers", doc);
    m.expert_stride = need_u64(root, "expertStride", doc);
    if (m.expert_stride % kAlignment != 0)
        raise(TF_ERR_ALIGNMENT, "manifest.expertStride %llu is not a multiple of %llu", (unsigned long long)m.expert_stride,
              (unsigned long long)kAlignment);
    if (m.model_id.empty() || m.experts_per_layer <= 0 || m.layers <= 0 || m.expert_stride == 0)
        raise(TF_ERR_FORMAT_INVALID, "manifest: invalid dimensions or stride");

    const Json& arch = need(root, "arch", Json::Object, doc);
    m.hidden = (int)need_int(arch, "hiddenSize", doc);
    m.ffn = (int)need_int(arch, "ffnIntermediate", doc);
    m.moe_ffn = (int)need_int(arch, "moeIntermediateSize", doc);
    m.num_layers = (int)need_int(arch, "numLayers", doc);
    m.num_experts = (int)need_int(arch, "numExperts", doc);
    m.top_k = (int)need_int(arch, "topKExperts", doc);
    m.vocab = (int)need_int(arch, "vocabSize", doc);
    m.activation = need(arch, "hiddenActivation", Json::String, doc).str;
    if (m.num_layers != m.layers || m.num_experts != m.experts_per_layer)
        raise(TF_ERR_FORMAT_INVALID, "manifest.arch: layer or expert count disagrees with the top-level fields");
    if (m.hidden <= 0 || m.ffn <= 0 || m.moe_ffn <= 0 || m.top_k <= 0 || m.top_k > m.num_experts || m.vocab <= 0)
        raise(TF_ERR_FORMAT_INVALID, "manifest.arch: invalid dimensions");

    if (const Json* quant = root.find("quant"); quant && quant->kind != Json::Null) {
        if (quant->kind != Json::Object) raise(TF_ERR_FORMAT_INVALID, "manifest.quant: not an object");
        m.has_quant = true;
        m.q_embedding = parse_slot(*quant, "embedding");
        m.q_attention = parse_slot(*quant, "attention");
        m.q_router = parse_slot(*quant, "router");
        m.q_shared = parse_slot(*quant, "sharedExpert");
        m.q_routed = parse_slot(*quant, "routedExpert");
        if (m.q_embedding.weight_bits != 4 || m.q_attention.weight_bits != 4 || m.q_router.weight_bits != 8 ||
            (m.q_shared.weight_bits != 4 && m.q_shared.weight_bits != 8) || m.q_routed.weight_bits != 4)
            raise(TF_ERR_FORMAT_INVALID, "manifest.quant: unsupported bit width");
    }

    const Json& files = need(root, "files", Json::Object, doc);
    std::set<std::string> keys;
    for (const auto& f : files.members) {
        const std::string field = "manifest.files." + f.first;
        validate_relative_path(f.first, field.c_str());
        if (!keys.insert(filesystem_key(f.first)).second)
            raise(TF_ERR_FORMAT_INVALID, "%s: collides with another entry on a case-insensitive file system", field.c_str());
        if (f.second.kind != Json::Object) raise(TF_ERR_FORMAT_INVALID, "%s: not an object", field.c_str());
        const std::string& sha = need(f.second, "sha256", Json::String, doc).str;
        bool hex = sha.size() == 64;
        for (char c : sha) hex = hex && ((c >= '0' && c <= '9') || (c >= 'a' && c <= 'f'));
        if (!hex) raise(TF_ERR_FORMAT_INVALID, "%s: sha256 is not 64 lower-case hex digits", field.c_str());
        m.file_sizes[f.first] = need_u64(f.second, "size", doc);
        m.file_sha256[f.first] = sha;
    }
    for (const char* required : {"model_weights.bin", "packed_experts/layout.json"})
        if (!m.file_sizes.count(required)) raise(TF_ERR_IO, "manifest.files: required entry %s is missing", required);
    return m;
}

Layout parse_layout(const char* bytes, size_t n) {
    const char* doc = "packed_experts/layout.json";
    const Json root = JsonParser(bytes, n, doc).parse();
    Layout lay;
    lay.expert_stride = need_u64(root, "expertStride", doc);
    lay.num_layers = (int)need_int(root, "numLayers", doc);
    lay.experts_per_layer = (int)need_int(root, "expertsPerLayer", doc);
    const Json& layers = need(root, "layers", Json::Array, doc);
    if (lay.num_layers <= 0 || lay.experts_per_layer <= 0 || lay.expert_stride == 0 || lay.expert_stride % kAlignment != 0 ||
        layers.items.size() != (size_t)lay.num_layers)
        raise(TF_ERR_FORMAT_INVALID, "layout: invalid dimensions or stride");
    std::set<int> layer_ids;
    std::set<std::string> layer_files;
    for (const Json& jl : layers.items) {
        Layer L;
        L.layer = (int)need_int(jl, "layer", doc);
        L.file = need(jl, "file", Json::String, doc).str;
        if (L.layer < 0 || L.layer >= lay.num_layers || !layer_ids.insert(L.layer).second)
            raise(TF_ERR_FORMAT_INVALID, "layout.layers: duplicate or invalid layer");
        const std::string field = "layout.layers[" + std::to_string(L.layer) + "]";
        validate_basename(L.file, (field + ".file").c_str());
        const std::string key = filesystem_key(L.file);
        if (key == "layout.json") raise(TF_ERR_FORMAT_INVALID, "%s.file: reserved packed-expert filename", field.c_str());
        if (!layer_files.insert(key).second) raise(TF_ERR_FORMAT_INVALID, "%s.file: duplicate layer filename", field.c_str());
        const Json& experts = need(jl, "experts", Json::Array, doc);
        if (experts.items.size() != (size_t)lay.experts_per_layer)
            raise(TF_ERR_FORMAT_INVALID, "%s.experts: wrong expert count", field.c_str());
        size_t explicit_ids = 0;
        for (const Json& je : experts.items) {
            int64_t tmp;
            if (optional_int(je, "expert", doc, &tmp)) ++explicit_ids;
        }
        if (explicit_ids != 0 && explicit_ids != experts.items.size())
            raise(TF_ERR_FORMAT_INVALID, "%s.experts: expert ids must be either all explicit or all positional", field.c_str());
        std::set<int> logical_ids, physical_ranks;
        std::set<uint64_t> offsets;
        int position = 0;
        for (const Json& je : experts.items) {
            Expert e;
            int64_t v;
            e.logical = optional_int(je, "expert", doc, &v) ? (int)v : position;
            e.physical = optional_int(je, "physicalRank", doc, &v) ? (int)v : e.logical;
            e.offset = need_u64(je, "offset", doc);
            e.size = need_u64(je, "size", doc);
            ++position;
            if (e.logical < 0 || e.logical >= lay.experts_per_layer || e.physical < 0 || e.physical >= lay.experts_per_layer ||
                !logical_ids.insert(e.logical).second || !physical_ranks.insert(e.physical).second ||
                !offsets.insert(e.offset).second)
                raise(TF_ERR_FORMAT_INVALID, "%s.experts: duplicate or invalid expert mapping", field.c_str());
            if (e.offset != checked_mul((uint64_t)e.physical, lay.expert_stride, "expert.offset") || e.size != lay.expert_stride)
                raise(TF_ERR_FORMAT_INVALID, "expert[%d]: offset or size does not match physical rank", e.logical);
            const Json& tensors = need(je, "tensors", Json::Object, doc);
            struct Range { uint64_t start, end; const std::string* name; };
            std::vector<Range> ranges;
            for (const auto& jt : tensors.members) {
                SubTensor t;
                t.offset = need_u64(jt.second, "offset", doc);
                t.size = need_u64(jt.second, "size", doc);
                t.dtype = need(jt.second, "dtype", Json::String, doc).str;
                for (const Json& d : need(jt.second, "shape", Json::Array, doc).items) {
                    if (d.kind != Json::Number || !d.is_uint || d.u > 0xFFFFFFFFull)
                        raise(TF_ERR_FORMAT_INVALID, "expert[%d].tensors.%s: invalid dtype or shape", e.logical, jt.first.c_str());
                    t.shape.push_back((uint32_t)d.u);
                }
                int64_t bits;
                const bool has_bits = optional_int(jt.second, "bits", doc, &bits);
                bool ok = (t.dtype == "U32" || t.dtype == "BF16") && !jt.first.empty() && t.size > 0 && !t.shape.empty();
                for (uint32_t d : t.shape) ok = ok && d > 0;
                if (has_bits) ok = ok && bits > 0 && bits <= 32;
                if (!ok) raise(TF_ERR_FORMAT_INVALID, "expert[%d].tensors.%s: invalid dtype or shape", e.logical, jt.first.c_str());
                t.bits = has_bits ? (int)bits : 0;
                const uint64_t end = checked_add(t.offset, t.size, "tensor.range");
                if (end > e.size) raise(TF_ERR_FORMAT_INVALID, "expert[%d].tensors.%s: range exceeds expert blob", e.logical, jt.first.c_str());
                auto placed = e.tensors.emplace(jt.first, std::move(t));
                ranges.push_back(Range{placed.first->second.offset, end, &placed.first->first});
            }
            std::sort(ranges.begin(), ranges.end(), [](const Range& a, const Range& b) {
                return a.start == b.start ? a.end < b.end : a.start < b.start;
            });
            for (size_t k = 1; k < ranges.size(); ++k)
                if (ranges[k - 1].end > ranges[k].start)
                    raise(TF_ERR_FORMAT_INVALID, "expert[%d].tensors: overlapping ranges %s and %s", e.logical,
                          ranges[k - 1].name->c_str(), ranges[k].name->c_str());
            L.experts.push_back(std::move(e));
        }
        std::sort(L.experts.begin(), L.experts.end(), [](const Expert& a, const Expert& b) { return a.logical < b.logical; });
        lay.layers.push_back(std::move(L));
    }
    std::sort(lay.layers.begin(), lay.layers.end(), [](const Layer& a, const Layer& b) { return a.layer < b.layer; });
    return lay;
}

void cross_validate(const Manifest& m, const Layout& lay) {
    if (m.layers != lay.num_layers || m.experts_per_layer != lay.experts_per_layer || m.expert_stride != lay.expert_stride)
        raise(TF_ERR_FORMAT_INVALID, "manifest/layout: dimension mismatch");
    const uint64_t layer_size = checked_mul((uint64_t)lay.experts_per_layer, lay.expert_stride, "layout.layerSize");
    for (const Layer& L : lay.layers) {
        const std::string path = "packed_experts/" + L.file;
        const auto it = m.file_sizes.find(path);
        if (it == m.file_sizes.end() || it->second != layer_size)
            raise(TF_ERR_FORMAT_INVALID, "manifest.files.%s: missing or wrong layer size", path.c_str());
    }
}

uint64_t rd(const uint8_t* p, int bytes) {
    uint64_t v = 0;
    for (int k = bytes - 1; k >= 0; --k) v = (v << 8) | p[k];     // little endian
    return v;
}

bool valid_utf8(const uint8_t* s, size_t n) {
    size_t k = 0;
    while (k < n) {
        const uint8_t c = s[k];
        size_t len;
        uint32_t cp;
        if (c < 0x80) { len = 1; cp = c; }
        else if ((c & 0xE0) == 0xC0) { len = 2; cp = c & 0x1F; }
        else if ((c & 0xF0) == 0xE0) { len = 3; cp = c & 0x0F; }
        else if ((c & 0xF8) == 0xF0) { len = 4; cp = c & 0x07; }
        else return false;
        if (k + len > n) return false;
        for (size_t j = 1; j < len; ++j) {
            if ((s[k + j] & 0xC0) != 0x80) return false;
            cp = (cp << 6) | (s[k + j] & 0x3F);
        }
        if ((len == 2 && cp < 0x80) || (len == 3 && cp < 0x800) || (len == 4 && cp < 0x10000) || cp > 0x10FFFF ||
            (cp >= 0xD800 && cp <= 0xDFFF))
            return false;
        k += len;
    }
    return true;
}

// `bytes` holds at least the index region (header, entries, names, padding) of model_weights.bin.
ResidentIndex parse_index(const uint8_t* bytes, size_t n) {
    if (n < kHeaderBytes) raise(TF_ERR_FORMAT_TRUNCATED, "resident.header: truncated");
    ResidentIndex idx;
    idx.index_size = rd(bytes, 8);
    idx.resident_size = rd(bytes + 8, 8);
    idx.entry_count = rd(bytes + 16, 8);
    if (idx.index_size > kIndexMaxBytes) raise(TF_ERR_FORMAT_INVALID, "resident.indexSize: exceeds v1 metadata cap");
    if (idx.index_size > n || idx.index_size < kHeaderBytes || idx.index_size % kAlignment != 0)
        raise(TF_ERR_FORMAT_TRUNCATED, "resident.index: truncated");
    const uint64_t table_bytes = checked_mul(idx.entry_count, kEntryBytes, "resident.entryTable");
    const uint64_t table_end = checked_add(kHeaderBytes, table_bytes, "resident.entryTable");
    if (table_end > idx.index_size) raise(TF_ERR_FORMAT_INVALID, "resident.entryTable: outside index");
    const uint64_t resident_end = checked_add(idx.index_size, idx.resident_size, "resident.payload");
    struct Range { uint64_t start, end; size_t entry; const char* what; };
    std::vector<Range> ranges;
    auto contained = [&](uint64_t off, uint64_t size, size_t entry, const char* what) {
        const uint64_t end = checked_add(off, size, what);
        if (off < idx.index_size || end > resident_end)
            raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].%s: range outside resident payload", entry, what);
        ranges.push_back(Range{off, end, entry, what});
    };
    for (size_t k = 0; k < (size_t)idx.entry_count; ++k) {
        const uint8_t* e = bytes + kHeaderBytes + k * kEntryBytes;
        const uint64_t name_off = rd(e, 4), name_len = rd(e + 4, 2);
        if (e[7] != 0) raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].reserved: must be zero", k);
        const uint64_t name_end = checked_add(name_off, name_len, "resident.entries.name");
        if (name_off < table_end || name_end > idx.index_size)
            raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].name: range outside string table", k);
        ResidentEntry r;
        r.name.assign(reinterpret_cast<const char*>(bytes + name_off), (size_t)name_len);
        if (r.name.empty() || !valid_utf8(bytes + name_off, (size_t)name_len) || idx.by_name.count(r.name))
            raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].name: invalid UTF-8 or duplicate", k);
        r.dtype = e[6];
        if (r.dtype > 3) raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].dtype: unknown dtype", k);
        r.file_offset = rd(e + 8, 8);
        r.size = rd(e + 16, 8);
        for (int d = 0; d < 4; ++d) r.shape[d] = (uint32_t)rd(e + 24 + 4 * d, 4);
        r.scale_offset = rd(e + 40, 8);
        r.scale_size = rd(e + 48, 8);
        r.bias_offset = rd(e + 56, 8);
        r.bias_size = rd(e + 64, 8);
        if (r.shape[0] == 0) raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].shape: first dimension must be positive", k);
        bool saw_zero = false;
        for (int d = 0; d < 4; ++d) {
            if (r.shape[d] == 0) saw_zero = true;
            else if (saw_zero) raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].shape: zero dimensions must be trailing", k);
        }
        if (r.size == 0) raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].weights: primary payload is empty", k);
        contained(r.file_offset, r.size, k, "weights");
        if (r.scale_size == 0) { if (r.scale_offset != 0) raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].scales: absent payload offset must be zero", k); }
        else contained(r.scale_offset, r.scale_size, k, "scales");
        if (r.bias_size == 0) { if (r.bias_offset != 0) raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].biases: absent payload offset must be zero", k); }
        else contained(r.bias_offset, r.bias_size, k, "biases");
        idx.by_name[r.name] = idx.entries.size();
        idx.entries.push_back(std::move(r));
    }
    std::sort(ranges.begin(), ranges.end(), [](const Range& a, const Range& b) {
        return a.start == b.start ? a.end < b.end : a.start < b.start;
    });
    for (size_t k = 1; k < ranges.size(); ++k)
        if (ranges[k].start < ranges[k - 1].end)
            raise(TF_ERR_FORMAT_INVALID, "resident.entries[%zu].%s: overlaps resident.entries[%zu].%s", ranges[k].entry,
                  ranges[k].what, ranges[k - 1].entry, ranges[k - 1].what);
    return idx;
}

// ---------------------------------------------------------------------------
// Files
// ---------------------------------------------------------------------------
struct Fd {
    int fd = -1;
    explicit Fd(const std::string& path) : fd(open(path.c_str(), O_RDONLY | O_CLOEXEC)) {
        if (fd < 0) raise(TF_ERR_IO, "open(%s): %s", path.c_str(), strerror(errno));
    }
    ~Fd() { if (fd >= 0) close(fd); }
    Fd(const Fd&) = delete;
    Fd& operator=(const Fd&) = delete;
    uint64_t size(const std::string& path) const {
        struct stat st;
        if (fstat(fd, &st) != 0) raise(TF_ERR_IO, "fstat(%s): %s", path.c_str(), strerror(errno));
        if (!S_ISREG(st.st_mode)) raise(TF_ERR_IO, "%s is not a regular file", path.c_str());
        return (uint64_t)st.st_size;
    }
    void read_exactly(void* dst, uint64_t bytes, uint64_t offset, const std::string& path) const {
        uint8_t* out = static_cast<uint8_t*>(dst);
        while (bytes > 0) {
            const ssize_t got = pread(fd, out, (size_t)std::min<uint64_t>(bytes, 1u << 30), (off_t)offset);
            if (got < 0) { if (errno == EINTR) continue; raise(TF_ERR_IO, "pread(%s): %s", path.c_str(), strerror(errno)); }
            if (got == 0) raise(TF_ERR_FORMAT_TRUNCATED, "%s: truncated at byte %llu", path.c_str(), (unsigned long long)offset);
            out += got; offset += (uint64_t)got; bytes -= (uint64_t)got;
        }
    }
};

std::vector<char> read_metadata(const std::string& path, uint64_t max_bytes) {
    Fd f(path);
    const uint64_t n = f.size(path);
    if (n > max_bytes) raise(TF_ERR_FORMAT_INVALID, "%s: %llu bytes exceed the metadata cap of %llu", path.c_str(),
                             (unsigned long long)n, (unsigned long long)max_bytes);
    std::vector<char> data((size_t)n);
    if (n) f.read_exactly(data.data(), n, 0, path);
    return data;
}

// Quantization.swift:17-28: bf16 <-> fp32, round to nearest even on the way down, no NaN special case.
float bf16_to_float(uint16_t bits) {
    const uint32_t w = (uint32_t)bits << 16;
    float f;
    memcpy(&f, &w, 4);
    return f;
}
uint16_t float_to_bf16(float f) {
    uint32_t w;
    memcpy(&w, &f, 4);
    const uint32_t rounding = 0x7FFFu + ((w >> 16) & 1u);
    return (uint16_t)((w + rounding) >> 16);
}

}  // namespace

struct tf_gturbo {
    std::string directory;        // empty when parsed from memory
    Manifest manifest;
    Layout layout;
    ResidentIndex index;
};

struct tf_gturbo_model {
    tf_context* ctx = nullptr;
    void* resident = nullptr;     // device copy of the resident payload
    uint64_t resident_bytes = 0;
    void* effective_scales = nullptr;   // bf16 [layers, hidden]
    std::vector<tf_moe_layer> layers;
};

namespace {

template <typename Fn>
tf_status guarded(const char* name, Fn&& fn) {
    try {
        fn();
        return TF_OK;
    } catch (const FormatError& e) {
        tf::set_global_error("%s: %s", name, e.text.c_str());
        return e.code;
    } catch (const std::bad_alloc&) {
        tf::set_global_error("%s: out of host memory", name);
        return TF_ERR_OUT_OF_MEMORY;
    }
}

const ResidentEntry& entry_named(const tf_gturbo& g, const std::string& name) {
    const auto it = g.index.by_name.find(name);
    if (it == g.index.by_name.end()) raise(TF_ERR_NOT_FOUND, "tensor %s is not in the resident index", name.c_str());
    return g.index.entries[it->second];
}

// Model.swift:195-233: absolute file offsets become offsets into the resident payload.
tf_gturbo_tensor view_of(const tf_gturbo& g, const ResidentEntry& e) {
    auto relative = [&](uint64_t absolute, uint64_t size, const char* what) -> uint64_t {
        if (size == 0) {
            if (absolute != 0) raise(TF_ERR_FORMAT_INVALID, "%s.%s has an absent nonzero offset", e.name.c_str(), what);
            return 0;
        }
        if (absolute < g.index.index_size) raise(TF_ERR_FORMAT_INVALID, "%s.%s precedes the resident payload", e.name.c_str(), what);
        const uint64_t rel = absolute - g.index.index_size;
        if (rel > g.index.resident_size || size > g.index.resident_size - rel)
            raise(TF_ERR_FORMAT_INVALID, "%s.%s exceeds the resident payload", e.name.c_str(), what);
        return rel;
    };
    tf_gturbo_tensor t;
    memset(&t, 0, sizeof t);
    t.dtype = e.dtype;
    t.offset = relative(e.file_offset, e.size, "weights");
    t.size = e.size;
    t.scale_offset = relative(e.scale_offset, e.scale_size, "scales");
    t.scale_size = e.scale_size;
    t.bias_offset = relative(e.bias_offset, e.bias_size, "biases");
    t.bias_size = e.bias_size;
    for (int d = 0; d < 4; ++d) t.shape[d] = e.shape[d];
    return t;
}

tf_expert_offsets expert_offsets_of(const tf_gturbo& g, uint32_t layer) {
    if (layer >= g.layout.layers.size()) raise(TF_ERR_INVALID_ARGUMENT, "layer %u out of range", layer);
    const Expert& e = g.layout.layers[layer].experts[0];
    auto off = [&](const char* role) -> uint32_t {
        const auto it = e.tensors.find(role);
        if (it == e.tensors.end() || it->second.offset > 0xFFFFFFFFull)
            raise(TF_ERR_FORMAT_INVALID, "invalid routed expert metadata for role %s", role);
        return (uint32_t)it->second.offset;
    };
    return tf_expert_offsets{off("gate"), off("gate_scales"), off("gate_biases"),
                             off("up"), off("up_scales"), off("up_biases"),
                             off("down"), off("down_scales"), off("down_biases")};
}

// One quantised resident matrix as a projection over the device copy of the payload; sizes are checked
// against rows x cols at the given bit width (group 64, 16-bit scale and bias per group).
tf_projection projection_of(const tf_gturbo& g, const void* device_base, const std::string& name, uint32_t rows, uint32_t cols,
                            int bits) {
    const tf_gturbo_tensor t = view_of(g, entry_named(g, name));
    const uint64_t w_bytes = (uint64_t)rows * cols * (uint64_t)bits / 8;
    const uint64_t sb_bytes = (uint64_t)rows * (cols / TF_GROUP_SIZE) * 2;
    if (cols % TF_GROUP_SIZE != 0 || t.size != w_bytes || t.scale_size != sb_bytes || t.bias_size != sb_bytes)
        raise(TF_ERR_DIMENSION_MISMATCH, "%s: expected %u x %u at %d bits (%llu + 2 x %llu bytes), found %llu + %llu + %llu",
              name.c_str(), rows, cols, bits, (unsigned long long)w_bytes, (unsigned long long)sb_bytes,
              (unsigned long long)t.size, (unsigned long long)t.scale_size, (unsigned long long)t.bias_size);
    tf_projection p;
    p.weights = device_base; p.weights_off = t.offset;
    p.scales = device_base;  p.scales_off = t.scale_offset;
    p.biases = device_base;  p.biases_off = t.bias_offset;
    p.rows = rows; p.cols = cols;
    return p;
}

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        raise(e == cudaErrorMemoryAllocation ? TF_ERR_OUT_OF_MEMORY : TF_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
}

}  // namespace

extern "C" {

tf_status tf_gturbo_parse(const void* manifest_json, uint64_t manifest_bytes, const void* layout_json, uint64_t layout_bytes,
                          const void* resident_index, uint64_t resident_index_bytes, tf_gturbo** out) {
    if (out) *out = nullptr;
    return guarded("tf_gturbo_parse", [&] {
        if (!out || !manifest_json || !layout_json || !resident_index) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        auto g = std::make_unique<tf_gturbo>();
        g->manifest = parse_manifest(static_cast<const char*>(manifest_json), (size_t)manifest_bytes);
        g->layout = parse_layout(static_cast<const char*>(layout_json), (size_t)layout_bytes);
        cross_validate(g->manifest, g->layout);
        g->index = parse_index(static_cast<const uint8_t*>(resident_index), (size_t)resident_index_bytes);
        *out = g.release();
    });
}

tf_status tf_gturbo_open(const char* directory, tf_gturbo** out) {
    if (out) *out = nullptr;
    return guarded("tf_gturbo_open", [&] {
        if (!out || !directory || !*directory) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        auto g = std::make_unique<tf_gturbo>();
        g->directory = directory;
        while (g->directory.size() > 1 && g->directory.back() == '/') g->directory.pop_back();
        const std::vector<char> manifest = read_metadata(g->directory + "/manifest.json", kManifestMaxBytes);
        g->manifest = parse_manifest(manifest.data(), manifest.size());
        const std::vector<char> layout = read_metadata(g->directory + "/packed_experts/layout.json", kLayoutMaxBytes);
        g->layout = parse_layout(layout.data(), layout.size());
        cross_validate(g->manifest, g->layout);

        const std::string weights = g->directory + "/model_weights.bin";
        Fd f(weights);
        const uint64_t file_bytes = f.size(weights);
        uint8_t header[kHeaderBytes];
        f.read_exactly(header, kHeaderBytes, 0, weights);
        const uint64_t index_size = rd(header, 8);
        if (index_size > kIndexMaxBytes) raise(TF_ERR_FORMAT_INVALID, "resident.indexSize: exceeds v1 metadata cap");
        if (index_size > file_bytes || index_size < kHeaderBytes) raise(TF_ERR_FORMAT_TRUNCATED, "resident.index: truncated");
        std::vector<uint8_t> region((size_t)index_size);
        f.read_exactly(region.data(), index_size, 0, weights);
        g->index = parse_index(region.data(), region.size());
        if (checked_add(g->index.index_size, g->index.resident_size, "resident.payload") > file_bytes)
            raise(TF_ERR_FORMAT_TRUNCATED, "%s: the resident payload extends beyond the file", weights.c_str());
        const auto listed = g->manifest.file_sizes.find("model_weights.bin");
        if (listed->second != file_bytes)
            raise(TF_ERR_FORMAT_INVALID, "model_weights.bin: %llu bytes on disk, %llu in the manifest",
                  (unsigned long long)file_bytes, (unsigned long long)listed->second);
        *out = g.release();
    });
}

void tf_gturbo_close(tf_gturbo* g) { delete g; }

tf_status tf_gturbo_get_info(const tf_gturbo* g, tf_gturbo_info* out) {
    return guarded("tf_gturbo_get_info", [&] {
        if (!g || !out) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        memset(out, 0, sizeof *out);
        out->version_major = (uint32_t)g->manifest.version_major;
        out->version_minor = (uint32_t)g->manifest.version_minor;
        out->num_layers = (uint32_t)g->manifest.layers;
        out->experts_per_layer = (uint32_t)g->manifest.experts_per_layer;
        out->top_k = (uint32_t)g->manifest.top_k;
        out->hidden_size = (uint32_t)g->manifest.hidden;
        out->moe_intermediate_size = (uint32_t)g->manifest.moe_ffn;
        out->ffn_intermediate = (uint32_t)g->manifest.ffn;
        out->shared_expert_bits = g->manifest.has_quant ? (uint32_t)g->manifest.q_shared.weight_bits : 0u;
        out->expert_stride = g->manifest.expert_stride;
        out->index_size = g->index.index_size;
        out->resident_size = g->index.resident_size;
        out->entry_count = g->index.entry_count;
    });
}

tf_status tf_gturbo_expert_offsets(const tf_gturbo* g, uint32_t layer, tf_expert_offsets* out) {
    return guarded("tf_gturbo_expert_offsets", [&] {
        if (!g || !out) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        *out = expert_offsets_of(*g, layer);
    });
}

tf_status tf_gturbo_expert_location(const tf_gturbo* g, uint32_t layer, uint32_t expert, const char** file_out,
                                    uint64_t* offset_out, uint64_t* size_out, uint32_t* physical_rank_out) {
    return guarded("tf_gturbo_expert_location", [&] {
        if (!g) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        if (layer >= g->layout.layers.size() || expert >= g->layout.layers[layer].experts.size())
            raise(TF_ERR_INVALID_ARGUMENT, "(layer %u, expert %u) out of range", layer, expert);
        const Expert& e = g->layout.layers[layer].experts[expert];
        if (file_out) *file_out = g->layout.layers[layer].file.c_str();
        if (offset_out) *offset_out = e.offset;
        if (size_out) *size_out = e.size;
        if (physical_rank_out) *physical_rank_out = (uint32_t)e.physical;
    });
}

tf_status tf_gturbo_resident(const tf_gturbo* g, const char* name, tf_gturbo_tensor* out) {
    return guarded("tf_gturbo_resident", [&] {
        if (!g || !name || !out) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        *out = view_of(*g, entry_named(*g, name));
    });
}

tf_status tf_gturbo_resident_name(const tf_gturbo* g, uint64_t position, const char** name_out) {
    return guarded("tf_gturbo_resident_name", [&] {
        if (!g || !name_out) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        if (position >= g->index.entries.size()) raise(TF_ERR_INVALID_ARGUMENT, "entry %llu out of range", (unsigned long long)position);
        *name_out = g->index.entries[(size_t)position].name.c_str();
    });
}

// Every blob of every layer file goes to its LOGICAL slot of the pool (the file stores experts by physical
// rank). A pool that holds a shard takes the experts [expert_offset, expert_offset + pool experts).
tf_status tf_expert_pool_load_gturbo(tf_pool* pool, void* stream, const tf_gturbo* g, uint32_t expert_offset) {
    return guarded("tf_expert_pool_load_gturbo", [&] {
        if (!pool || !g) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        if (g->directory.empty()) raise(TF_ERR_INVALID_ARGUMENT, "the handle was parsed from memory and has no directory");
        uint32_t layers = 0, experts = 0;
        uint64_t stride = 0;
        tf_expert_pool_dims(pool, &layers, &experts, &stride);
        if (layers != (uint32_t)g->layout.num_layers || stride != g->layout.expert_stride ||
            (uint64_t)expert_offset + experts > (uint64_t)g->layout.experts_per_layer)
            raise(TF_ERR_DIMENSION_MISMATCH, "pool of %u layers x %u experts (from %u) x %llu bytes does not fit a model of %d x %d x %llu",
                  layers, experts, expert_offset, (unsigned long long)stride, g->layout.num_layers, g->layout.experts_per_layer,
                  (unsigned long long)g->layout.expert_stride);
        // Two pinned staging buffers: the read of blob k + 1 overlaps the copy of blob k.
        void* staging[2] = {nullptr, nullptr};
        cudaEvent_t done[2] = {nullptr, nullptr};
        struct Cleanup {
            void** s; cudaEvent_t* d;
            ~Cleanup() { for (int k = 0; k < 2; ++k) { if (d[k]) cudaEventDestroy(d[k]); if (s[k]) cudaFreeHost(s[k]); } }
        } cleanup{staging, done};
        for (int k = 0; k < 2; ++k) {
            cuda_check(cudaHostAlloc(&staging[k], stride, cudaHostAllocDefault), "cudaHostAlloc(staging)");
            cuda_check(cudaEventCreateWithFlags(&done[k], cudaEventDisableTiming), "cudaEventCreate");
        }
        const uint64_t layer_bytes = checked_mul((uint64_t)g->layout.experts_per_layer, stride, "layout.layerSize");
        uint64_t turn = 0;
        for (const Layer& L : g->layout.layers) {
            const std::string path = g->directory + "/packed_experts/" + L.file;
            Fd f(path);
            if (f.size(path) != layer_bytes)
                raise(TF_ERR_FORMAT_INVALID, "%s: %llu bytes on disk, expected %llu", path.c_str(),
                      (unsigned long long)f.size(path), (unsigned long long)layer_bytes);
            for (uint32_t slot = 0; slot < experts; ++slot, ++turn) {
                const Expert& e = L.experts[expert_offset + slot];
                const int b = (int)(turn & 1);
                if (turn >= 2) cuda_check(cudaEventSynchronize(done[b]), "cudaEventSynchronize");
                f.read_exactly(staging[b], stride, e.offset, path);
                const tf_status st = tf_expert_pool_upload(pool, stream, (uint32_t)L.layer, slot, staging[b], stride);
                if (st != TF_OK) raise(st, "upload of layer %d expert %d failed: %s", L.layer, e.logical, tf_last_error(nullptr));
                cuda_check(cudaEventRecord(done[b], static_cast<cudaStream_t>(stream)), "cudaEventRecord");
            }
        }
        cuda_check(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "cudaStreamSynchronize");
    });
}

// Upload of the resident payload and the per-layer views the MoE block needs. Tensor names are the
// checkpoint's (Runtime/Inference/Model.swift:89-188).
tf_status tf_gturbo_model_load(tf_context* ctx, void* stream, const tf_gturbo* g, const tf_pool* pool, tf_gturbo_model** out) {
    if (out) *out = nullptr;
    return guarded("tf_gturbo_model_load", [&] {
        if (!ctx || !g || !pool || !out) raise(TF_ERR_INVALID_ARGUMENT, "NULL argument");
        if (g->directory.empty()) raise(TF_ERR_INVALID_ARGUMENT, "the handle was parsed from memory and has no directory");
        const Manifest& m = g->manifest;
        const int shared_bits = m.has_quant ? m.q_shared.weight_bits : 4;
        if (shared_bits != 4 && shared_bits != 8)
            raise(TF_ERR_UNSUPPORTED, "shared expert at %d bits: the block kernels take a 4-bit or an 8-bit shared expert", shared_bits);
        uint32_t pool_layers = 0, pool_experts = 0;
        uint64_t pool_stride = 0;
        tf_expert_pool_dims(pool, &pool_layers, &pool_experts, &pool_stride);
        if (pool_layers != (uint32_t)m.layers || pool_experts != (uint32_t)m.experts_per_layer || pool_stride != m.expert_stride)
            raise(TF_ERR_DIMENSION_MISMATCH, "the pool does not hold every expert of this model");

        auto model = std::make_unique<tf_gturbo_model>();
        model->ctx = ctx;
        struct Guard {
            tf_gturbo_model* m; bool keep = false;
            ~Guard() { if (!keep) { if (m->resident) cudaFree(m->resident); if (m->effective_scales) cudaFree(m->effective_scales); } }
        } guard{model.get()};
        model->resident_bytes = g->index.resident_size;
        cuda_check(cudaMalloc(&model->resident, std::max<uint64_t>(model->resident_bytes, 256)), "cudaMalloc(resident payload)");
        const std::string weights = g->directory + "/model_weights.bin";
        Fd f(weights);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        {
            constexpr uint64_t kChunk = 64u << 20;
            std::vector<uint8_t> chunk((size_t)std::min<uint64_t>(kChunk, std::max<uint64_t>(model->resident_bytes, 1)));
            for (uint64_t done = 0; done < model->resident_bytes; done += kChunk) {
                const uint64_t n = std::min<uint64_t>(kChunk, model->resident_bytes - done);
                f.read_exactly(chunk.data(), n, g->index.index_size + done, weights);
                // pageable source: the call returns once the bytes are staged, so the chunk can be refilled
                cuda_check(cudaMemcpyAsync(static_cast<uint8_t*>(model->resident) + done, chunk.data(), n, cudaMemcpyHostToDevice, s),
                           "cudaMemcpyAsync(resident payload)");
                cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
            }
        }

        const uint32_t D = (uint32_t)m.hidden, F = (uint32_t)m.moe_ffn, Fs = (uint32_t)m.ffn, E = (uint32_t)m.num_experts;
        // router.scale x 1/sqrt(D), rounded to bf16 once per layer (RealForwardRunner.swift:352-376)
        std::vector<uint16_t> eff((size_t)m.layers * D);
        const float inv_sqrt_d = 1.0f / std::sqrt((float)D);
        std::vector<uint16_t> scale(D);
        for (int L = 0; L < m.layers; ++L) {
            const std::string prefix = "language_model.model.layers." + std::to_string(L);
            const ResidentEntry& e = entry_named(*g, prefix + ".router.scale");
            if (e.dtype != 1 || e.size != (uint64_t)D * 2) raise(TF_ERR_DIMENSION_MISMATCH, "%s: expected bf16[%u]", e.name.c_str(), D);
            f.read_exactly(scale.data(), e.size, e.file_offset, weights);
            for (uint32_t k = 0; k < D; ++k) eff[(size_t)L * D + k] = float_to_bf16(bf16_to_float(scale[k]) * inv_sqrt_d);
        }
        cuda_check(cudaMalloc(&model->effective_scales, eff.size() * 2), "cudaMalloc(effective scales)");
        cuda_check(cudaMemcpyAsync(model->effective_scales, eff.data(), eff.size() * 2, cudaMemcpyHostToDevice, s), "cudaMemcpyAsync");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");

        for (int L = 0; L < m.layers; ++L) {
            const std::string prefix = "language_model.model.layers." + std::to_string(L);
            tf_moe_layer layer;
            memset(&layer, 0, sizeof layer);
            layer.router = projection_of(*g, model->resident, prefix + ".router.proj.weight", E, D, 8);
            layer.effective_scale = static_cast<const uint16_t*>(model->effective_scales) + (size_t)L * D;
            const ResidentEntry& pes = entry_named(*g, prefix + ".router.per_expert_scale");
            if (pes.dtype != 1 || pes.size != (uint64_t)E * 2) raise(TF_ERR_DIMENSION_MISMATCH, "%s: expected bf16[%u]", pes.name.c_str(), E);
            layer.per_expert_scale = static_cast<const uint8_t*>(model->resident) + view_of(*g, pes).offset;
            layer.logit_bias = nullptr;
            layer.pool_layer_base = tf_expert_pool_ptr(pool, (uint32_t)L, 0);
            layer.expert_stride = m.expert_stride;
            layer.offsets = expert_offsets_of(*g, (uint32_t)L);
            layer.shared_gate = projection_of(*g, model->resident, prefix + ".mlp.gate_proj.weight", Fs, D, shared_bits);
            layer.shared_up = projection_of(*g, model->resident, prefix + ".mlp.up_proj.weight", Fs, D, shared_bits);
            layer.shared_down = projection_of(*g, model->resident, prefix + ".mlp.down_proj.weight", D, Fs, shared_bits);
            layer.num_experts = E; layer.d = D; layer.f = F; layer.fs = Fs; layer.top_k = (uint32_t)m.top_k;
            layer.shared_bits = (uint32_t)shared_bits;
            model->layers.push_back(layer);
        }
        guard.keep = true;
        *out = model.release();
    });
}

void tf_gturbo_model_destroy(tf_gturbo_model* model) {
    if (!model) return;
    if (model->resident) cudaFree(model->resident);
    if (model->effective_scales) cudaFree(model->effective_scales);
    delete model;
}

const tf_moe_layer* tf_gturbo_model_layers(const tf_gturbo_model* model, uint32_t* count_out) {
    if (count_out) *count_out = model ? (uint32_t)model->layers.size() : 0u;
    return model && !model->layers.empty() ? model->layers.data() : nullptr;
}

const void* tf_gturbo_model_resident_base(const tf_gturbo_model* model) { return model ? model->resident : nullptr; }

}  // extern "C"
