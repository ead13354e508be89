// MLX 4-bit checkpoints -> Q4 banks: the on-disk side of the path.
//
// Mirrors the part of the reference's loader that produces a `Q4MlxBank`
// (src/loader.rs:236-318 `mlx_q4_named`, src/qwen35_q4.rs:204-255 `MlxQuant::from_config_json`,
// 378-381 `sidecar_names`, 384-449 `check_part` of the reference project):
//   * a strict reader of the safetensors container (8-byte little-endian header length, a JSON
//     object of name -> {dtype, shape, data_offsets}, then the tensor bytes); the reference takes
//     this from a crate that is not in its tree, so it is written here from the format;
//   * `config.json`'s `quantization` object: only uniform affine, 4 bits, group 64 is accepted;
//   * one quantized matrix = `X.weight` U32 [rows, cols / 8] + `X.scales`, `X.biases` BF16
//     [rows, cols / 64], each checked against its header before any byte is read;
//   * a bank = the rows of several such matrices one after the other (q/k/v, gate/up), the packed
//     words copied unchanged, scales and biases interleaved into (scale, bias) pairs, and a
//     non-finite scale or bias refused by tensor, row and group.
// Everything but the final upload is host code and runs without a GPU. Which tensors make up
// which projection (the model's naming) is the caller's business, as in the reference, where
// `Loader::mlx_q4` is handed the part names.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <thread>
#include <vector>

#include "runtime.h"

namespace tessl {
namespace {

constexpr uint32_t kMlxQ4Bits = 4, kMlxQ4Group = 64, kNibblesPerWord = 8;

// ------------------------------------------------------------------ JSON ---

struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    bool integral = false;  // a number written without fraction or exponent
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;  // insertion order; duplicate keys are refused

    const Json *get(const std::string &key) const
    {
        for (const auto &kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool operator==(const Json &o) const
    {
        if (kind != o.kind) return false;
        switch (kind) {
        case Null: return true;
        case Bool: return b == o.b;
        case Number: return num == o.num;
        case String: return str == o.str;
        case Array: return arr == o.arr;
        case Object: {
            if (obj.size() != o.obj.size()) return false;
            for (const auto &kv : obj) {
                const Json *other = o.get(kv.first);
                if (!other || !(*other == kv.second)) return false;
            }
            return true;
        }
        }
        return false;
    }
};

class JsonParser {
public:
    JsonParser(const char *p, size_t n) : p_(p), end_(p + n) {}
    Result parse(Json *out)
    {
        TESSL_TRY(value(out, 0));
        ws();
        if (p_ != end_) return "trailing characters after the JSON value";
        return ok();
    }

private:
    const char *p_, *end_;
    void ws()
    {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    Result value(Json *out, int depth)
    {
        if (depth > 64) return "JSON nested deeper than 64 levels";
        ws();
        if (p_ >= end_) return "unexpected end of JSON";
        const char c = *p_;
        if (c == '{') return object(out, depth);
        if (c == '[') return array(out, depth);
        if (c == '"') {
            out->kind = Json::String;
            return string(&out->str);
        }
        if (c == 't' || c == 'f' || c == 'n') return literal(out);
        if (c == '-' || (c >= '0' && c <= '9')) return number(out);
        return fmt("unexpected character '%c' in JSON", c);
    }
    Result literal(Json *out)
    {
        auto take = [&](const char *w) {
            const size_t n = std::strlen(w);
            if ((size_t)(end_ - p_) >= n && std::memcmp(p_, w, n) == 0) {
                p_ += n;
                return true;
            }
            return false;
        };
        if (take("true")) return out->kind = Json::Bool, out->b = true, ok();
        if (take("false")) return out->kind = Json::Bool, out->b = false, ok();
        if (take("null")) return out->kind = Json::Null, ok();
        return "malformed JSON literal";
    }
    Result number(Json *out)
    {
        const char *s = p_;
        if (p_ < end_ && *p_ == '-') ++p_;
        if (p_ >= end_ || *p_ < '0' || *p_ > '9') return "malformed JSON number";
        if (*p_ == '0') {
            ++p_;
        } else {
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        bool integral = true;
        if (p_ < end_ && *p_ == '.') {
            integral = false;
            ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') return "malformed JSON number";
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        if (p_ < end_ && (*p_ == 'e' || *p_ == 'E')) {
            integral = false;
            ++p_;
            if (p_ < end_ && (*p_ == '+' || *p_ == '-')) ++p_;
            if (p_ >= end_ || *p_ < '0' || *p_ > '9') return "malformed JSON number";
            while (p_ < end_ && *p_ >= '0' && *p_ <= '9') ++p_;
        }
        out->kind = Json::Number;
        out->integral = integral;
        out->num = std::strtod(std::string(s, p_).c_str(), nullptr);
        return ok();
    }
    Result string(std::string *out)
    {
        ++p_;  // opening quote
        out->clear();
        while (true) {
            if (p_ >= end_) return "unterminated JSON string";
            const unsigned char c = (unsigned char)*p_++;
            if (c == '"') return ok();
            if (c < 0x20) return "control character in JSON string";
            if (c != '\\') {
                out->push_back((char)c);
                continue;
            }
            if (p_ >= end_) return "unterminated JSON escape";
            const char e = *p_++;
            switch (e) {
            case '"': out->push_back('"'); break;
            case '\\': out->push_back('\\'); break;
            case '/': out->push_back('/'); break;
            case 'b': out->push_back('\b'); break;
            case 'f': out->push_back('\f'); break;
            case 'n': out->push_back('\n'); break;
            case 'r': out->push_back('\r'); break;
            case 't': out->push_back('\t'); break;
            case 'u': {
                if (end_ - p_ < 4) return "truncated \\u escape";
                unsigned cp = 0;
                for (int i = 0; i < 4; ++i) {
                    const char h = *p_++;
                    cp <<= 4;
                    if (h >= '0' && h <= '9') cp |= (unsigned)(h - '0');
                    else if (h >= 'a' && h <= 'f') cp |= (unsigned)(h - 'a' + 10);
                    else if (h >= 'A' && h <= 'F') cp |= (unsigned)(h - 'A' + 10);
                    else return "malformed \\u escape";
                }
                // tensor names are ASCII in practice; encode the BMP code point as UTF-8 (surrogates refused)
                if (cp >= 0xD800 && cp <= 0xDFFF) return "surrogate \\u escape in JSON string";
                if (cp < 0x80) {
                    out->push_back((char)cp);
                } else if (cp < 0x800) {
                    out->push_back((char)(0xC0 | (cp >> 6))), out->push_back((char)(0x80 | (cp & 0x3F)));
                } else {
                    out->push_back((char)(0xE0 | (cp >> 12))), out->push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
                    out->push_back((char)(0x80 | (cp & 0x3F)));
                }
                break;
            }
            default: return "unknown escape in JSON string";
            }
        }
    }
    Result array(Json *out, int depth)
    {
        ++p_;
        out->kind = Json::Array;
        ws();
        if (p_ < end_ && *p_ == ']') return ++p_, ok();
        while (true) {
            out->arr.emplace_back();
            TESSL_TRY(value(&out->arr.back(), depth + 1));
            ws();
            if (p_ >= end_) return "unterminated JSON array";
            if (*p_ == ',') {
                ++p_;
                continue;
            }
            if (*p_ == ']') return ++p_, ok();
            return "expected ',' or ']' in JSON array";
        }
    }
    Result object(Json *out, int depth)
    {
        ++p_;
        out->kind = Json::Object;
        ws();
        if (p_ < end_ && *p_ == '}') return ++p_, ok();
        while (true) {
            ws();
            if (p_ >= end_ || *p_ != '"') return "expected a string key in JSON object";
            std::string key;
            TESSL_TRY(string(&key));
            if (out->get(key)) return fmt("duplicate key \"%s\" in JSON object", key.c_str());
            ws();
            if (p_ >= end_ || *p_ != ':') return "expected ':' in JSON object";
            ++p_;
            out->obj.emplace_back(key, Json());
            TESSL_TRY(value(&out->obj.back().second, depth + 1));
            ws();
            if (p_ >= end_) return "unterminated JSON object";
            if (*p_ == ',') {
                ++p_;
                continue;
            }
            if (*p_ == '}') return ++p_, ok();
            return "expected ',' or '}' in JSON object";
        }
    }
};

std::string describe(const Json &v)
{
    switch (v.kind) {
    case Json::Null: return "null";
    case Json::Bool: return v.b ? "true" : "false";
    case Json::Number: return fmt("%g", v.num);
    case Json::String: return "\"" + v.str + "\"";
    case Json::Array: return "an array";
    case Json::Object: return "an object";
    }
    return "?";
}

// ----------------------------------------------------------- safetensors ---

struct TensorEntry {
    std::string dtype;
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;  // byte range within the data section
};

size_t dtype_size(const std::string &d)
{
    if (d == "BOOL" || d == "U8" || d == "I8" || d == "F8_E4M3" || d == "F8_E5M2") return 1;
    if (d == "U16" || d == "I16" || d == "F16" || d == "BF16") return 2;
    if (d == "U32" || d == "I32" || d == "F32") return 4;
    if (d == "U64" || d == "I64" || d == "F64") return 8;
    return 0;
}

std::string shape_text(const std::vector<uint64_t> &s)
{
    std::string t = "[";
    for (size_t i = 0; i < s.size(); ++i) t += (i ? ", " : "") + std::to_string(s[i]);
    return t + "]";
}

}  // namespace
}  // namespace tessl

struct TesslCheckpoint {
    std::string path;
    const uint8_t *map = nullptr;
    size_t map_len = 0;
    const uint8_t *data = nullptr;  // start of the tensor bytes
    size_t data_len = 0;
    std::vector<std::string> names;  // header order
    std::map<std::string, tessl::TensorEntry> tensors;

    ~TesslCheckpoint()
    {
        if (map) munmap(const_cast<uint8_t *>(map), map_len);
    }
};

namespace tessl {
namespace {

Result open_checkpoint(const char *path, std::unique_ptr<TesslCheckpoint> *out)
{
    if (!path) return "checkpoint: null path";
    auto ck = std::make_unique<TesslCheckpoint>();
    ck->path = path;
    const int fd = ::open(path, O_RDONLY);
    if (fd < 0) return fmt("%s: cannot open (%s)", path, std::strerror(errno));
    struct stat st {};
    if (fstat(fd, &st) != 0 || st.st_size < 8) {
        ::close(fd);
        return fmt("%s: shorter than a safetensors header", path);
    }
    ck->map_len = (size_t)st.st_size;
    void *m = mmap(nullptr, ck->map_len, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) {
        ck->map_len = 0;
        return fmt("%s: cannot map (%s)", path, std::strerror(errno));
    }
    ck->map = static_cast<const uint8_t *>(m);
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | ck->map[i];
    if (hlen > ck->map_len - 8) return fmt("%s: header length %llu exceeds the file", path, (unsigned long long)hlen);
    if (hlen > (100ull << 20)) return fmt("%s: header length %llu exceeds 100 MiB", path, (unsigned long long)hlen);
    Json root;
    {
        Result r = JsonParser(reinterpret_cast<const char *>(ck->map + 8), (size_t)hlen).parse(&root);
        if (!r.empty()) return fmt("%s: header: %s", path, r.c_str());
    }
    if (root.kind != Json::Object) return fmt("%s: header is not a JSON object", path);
    ck->data = ck->map + 8 + hlen;
    ck->data_len = ck->map_len - 8 - (size_t)hlen;
    std::vector<std::pair<uint64_t, uint64_t>> ranges;
    for (const auto &kv : root.obj) {
        if (kv.first == "__metadata__") {
            if (kv.second.kind != Json::Object) return fmt("%s: __metadata__ is not an object", path);
            continue;
        }
        const Json &t = kv.second;
        if (t.kind != Json::Object) return fmt("%s: %s: entry is not an object", path, kv.first.c_str());
        const Json *dt = t.get("dtype"), *sh = t.get("shape"), *off = t.get("data_offsets");
        if (!dt || dt->kind != Json::String) return fmt("%s: %s: no dtype string", path, kv.first.c_str());
        if (!sh || sh->kind != Json::Array) return fmt("%s: %s: no shape array", path, kv.first.c_str());
        if (!off || off->kind != Json::Array || off->arr.size() != 2)
            return fmt("%s: %s: data_offsets is not a pair", path, kv.first.c_str());
        TensorEntry e;
        e.dtype = dt->str;
        const size_t esz = dtype_size(e.dtype);
        if (esz == 0) return fmt("%s: %s: unknown dtype %s", path, kv.first.c_str(), e.dtype.c_str());
        auto uint_of = [](const Json &v, uint64_t *o) {
            if (v.kind != Json::Number || !v.integral || v.num < 0.0 || v.num > 9007199254740992.0) return false;
            *o = (uint64_t)v.num;
            return true;
        };
        uint64_t count = 1;
        for (const Json &d : sh->arr) {
            uint64_t v = 0;
            if (!uint_of(d, &v)) return fmt("%s: %s: shape holds %s", path, kv.first.c_str(), describe(d).c_str());
            if (v != 0 && count > (1ull << 62) / v) return fmt("%s: %s: shape overflows", path, kv.first.c_str());
            count *= v;
            e.shape.push_back(v);
        }
        if (!uint_of(off->arr[0], &e.begin) || !uint_of(off->arr[1], &e.end) || e.begin > e.end)
            return fmt("%s: %s: malformed data_offsets", path, kv.first.c_str());
        if (e.end > ck->data_len)
            return fmt("%s: %s: data_offsets %llu..%llu exceed the %zu bytes of tensor data", path, kv.first.c_str(),
                       (unsigned long long)e.begin, (unsigned long long)e.end, ck->data_len);
        if (e.end - e.begin != count * esz)
            return fmt("%s: %s: %s %s needs %llu bytes, data_offsets give %llu", path, kv.first.c_str(), e.dtype.c_str(),
                       shape_text(e.shape).c_str(), (unsigned long long)(count * esz), (unsigned long long)(e.end - e.begin));
        if (e.end > e.begin) ranges.emplace_back(e.begin, e.end);
        ck->names.push_back(kv.first);
        ck->tensors.emplace(kv.first, std::move(e));
    }
    std::sort(ranges.begin(), ranges.end());
    for (size_t i = 1; i < ranges.size(); ++i)
        if (ranges[i].first < ranges[i - 1].second) return fmt("%s: two tensors' data_offsets overlap", path);
    *out = std::move(ck);
    return ok();
}

Result find(const TesslCheckpoint &ck, const std::string &name, const TensorEntry **out)
{
    auto it = ck.tensors.find(name);
    if (it == ck.tensors.end()) return fmt("%s: no such tensor in %s", name.c_str(), ck.path.c_str());
    *out = &it->second;
    return ok();
}

/// `sidecar_names` (src/qwen35_q4.rs:378-381).
bool sidecar_names(const std::string &weight, std::string *scales, std::string *biases)
{
    const std::string suffix = ".weight";
    if (weight.size() < suffix.size() || weight.compare(weight.size() - suffix.size(), suffix.size(), suffix) != 0) return false;
    const std::string base = weight.substr(0, weight.size() - suffix.size());
    *scales = base + ".scales", *biases = base + ".biases";
    return true;
}

/// `check_part` (src/qwen35_q4.rs:384-449), same order of refusals and wording of `MlxQ4Error`'s Display.
Result check_part(const TesslCheckpoint &ck, const std::string &weight_name, uint64_t rows, uint64_t cols)
{
    const TensorEntry *w = nullptr;
    TESSL_TRY(find(ck, weight_name, &w));
    if (rows == 0 || cols == 0)
        return fmt("%s: a [%llu, %llu] matrix has nothing to load", weight_name.c_str(), (unsigned long long)rows,
                   (unsigned long long)cols);
    if (cols % kMlxQ4Group != 0 || cols % kNibblesPerWord != 0)
        return fmt("%s: %llu columns is not a multiple of the group size %u", weight_name.c_str(), (unsigned long long)cols,
                   kMlxQ4Group);
    if (w->dtype != "U32")
        return fmt("%s: a %s tensor in a quantized checkpoint (a layer the converter left dense); a mixed checkpoint is "
                   "not supported", weight_name.c_str(), w->dtype.c_str());
    const std::vector<uint64_t> want_w = {rows, cols / kNibblesPerWord};
    if (w->shape != want_w)
        return fmt("%s: shape %s, expected %s (4-bit packs eight values per U32 word; a different width means other bits)",
                   weight_name.c_str(), shape_text(w->shape).c_str(), shape_text(want_w).c_str());
    std::string sn, bn;
    if (!sidecar_names(weight_name, &sn, &bn))
        return fmt("%s: dtype a name that does not end in .weight, expected X.weight", weight_name.c_str());
    const std::pair<const std::string *, const char *> sides[2] = {{&sn, "scales"}, {&bn, "biases"}};
    for (const auto &side : sides) {
        auto it = ck.tensors.find(*side.first);
        if (it == ck.tensors.end())
            return fmt("%s: packed 4-bit weight with no %s tensor beside it", weight_name.c_str(), side.second);
        const TensorEntry &e = it->second;
        if (e.dtype != "BF16")
            return fmt("%s: dtype %s, expected BF16 (a bf16 model's scales; float16 checkpoints are not supported)",
                       side.first->c_str(), e.dtype.c_str());
        const std::vector<uint64_t> want = {rows, cols / kMlxQ4Group};
        if (e.shape != want)
            return fmt("%s: shape %s, expected %s (4-bit packs eight values per U32 word; a different width means other bits)",
                       side.first->c_str(), shape_text(e.shape).c_str(), shape_text(want).c_str());
    }
    return ok();
}

/// `Loader::mlx_q4_named` (src/loader.rs:256-318) into host memory: every part's headers first, then the
/// packed words unchanged and the scale/bias pairs interleaved, rows of the parts one after the other.
Result read_bank(const TesslCheckpoint &ck, const char *const *names, const uint64_t *rows, uint32_t nparts, uint64_t cols,
                 uint8_t *packed, uint64_t packed_bytes, uint16_t *pairs, uint64_t pairs_bytes)
{
    if (nparts == 0) return "mlx_q4: no parts";
    uint64_t total = 0;
    for (uint32_t i = 0; i < nparts; ++i) {
        if (!names[i]) return "mlx_q4: null part name";
        if (rows[i] > (1ull << 40) || total + rows[i] < total) return "mlx_q4: output widths overflow";
        total += rows[i];
    }
    for (uint32_t i = 0; i < nparts; ++i) TESSL_TRY(check_part(ck, names[i], rows[i], cols));
    const uint64_t groups = cols / kMlxQ4Group, row_bytes = cols / 2;
    if (packed_bytes < total * row_bytes)
        return fmt("mlx_q4: the packed buffer holds %llu bytes, the bank needs %llu", (unsigned long long)packed_bytes,
                   (unsigned long long)(total * row_bytes));
    if (pairs_bytes < total * groups * 4)
        return fmt("mlx_q4: the scale/bias buffer holds %llu bytes, the bank needs %llu", (unsigned long long)pairs_bytes,
                   (unsigned long long)(total * groups * 4));
    uint64_t row0 = 0;
    for (uint32_t i = 0; i < nparts; ++i) {
        const TensorEntry *w = nullptr, *s = nullptr, *b = nullptr;
        std::string sn, bn;
        sidecar_names(names[i], &sn, &bn);
        TESSL_TRY(find(ck, names[i], &w));
        TESSL_TRY(find(ck, sn, &s));
        TESSL_TRY(find(ck, bn, &b));
        std::memcpy(packed + row0 * row_bytes, ck.data + w->begin, (size_t)(rows[i] * row_bytes));
        const uint16_t *sc = reinterpret_cast<const uint16_t *>(ck.data + s->begin);  // may be unaligned: read by memcpy
        const uint16_t *bi = reinterpret_cast<const uint16_t *>(ck.data + b->begin);
        const uint64_t n = rows[i] * groups;
        uint16_t *dst = pairs + 2 * row0 * groups;
        for (uint64_t k = 0; k < n; ++k) {
            uint16_t sv, bv;
            std::memcpy(&sv, reinterpret_cast<const uint8_t *>(sc) + 2 * k, 2);
            std::memcpy(&bv, reinterpret_cast<const uint8_t *>(bi) + 2 * k, 2);
            // a bf16 with every exponent bit set is an infinity or a NaN (src/loader.rs:296-308)
            for (int which = 0; which < 2; ++which) {
                const uint16_t bits = which ? bv : sv;
                if ((bits & 0x7f80u) == 0x7f80u) {
                    const uint32_t f32 = (uint32_t)bits << 16;
                    float val;
                    std::memcpy(&val, &f32, 4);
                    return fmt("%s: element %llu (row %llu, group %llu) is %s, not finite", (which ? bn : sn).c_str(),
                               (unsigned long long)k, (unsigned long long)(k / groups), (unsigned long long)(k % groups),
                               std::isnan(val) ? "NaN" : (val > 0 ? "inf" : "-inf"));
                }
            }
            dst[2 * k] = sv, dst[2 * k + 1] = bv;
        }
        row0 += rows[i];
    }
    return ok();
}

/// `MlxQuant::from_config_json` (src/qwen35_q4.rs:204-255).
Result quant_from_config_json(const char *text, uint32_t *bits, uint32_t *group_size)
{
    if (!text) return "config.json: null text";
    Json root;
    {
        Result r = JsonParser(text, std::strlen(text)).parse(&root);
        if (!r.empty()) return fmt("config.json: quantization.config.json: %s", r.c_str());
    }
    if (root.kind != Json::Object) return "config.json: quantization.config.json: not a JSON object";
    const Json *a = root.get("quantization"), *b = root.get("quantization_config");
    if (!a && !b) return "config.json: no \"quantization\" object; this is not an MLX-quantized checkpoint";
    if (a && b && !(*a == *b)) return "config.json: quantization.quantization_config: differs from quantization";
    const Json &q = a ? *a : *b;
    if (q.kind != Json::Object)
        return fmt("config.json: quantization.quantization: must be an object, got %s", describe(q).c_str());
    std::string overrides;
    for (const auto &kv : q.obj) {
        if (kv.first != "group_size" && kv.first != "bits" && kv.first != "mode")
            overrides += (overrides.empty() ? "\"" : ", \"") + kv.first + "\"";
    }
    if (!overrides.empty())
        return fmt("config.json: quantization has per-layer entries [%s]: a mixed-precision checkpoint (other bits, or layers "
                   "left dense) is not supported; only one uniform affine group-64 4-bit quantization", overrides.c_str());
    auto uint_key = [&](const char *k, uint32_t *out) -> Result {
        const Json *v = q.get(k);
        if (!v) return fmt("config.json: quantization.%s: missing", k);
        if (v->kind != Json::Number || !v->integral || v->num < 0.0 || v->num > 4294967295.0)
            return fmt("config.json: quantization.%s: must be an unsigned integer, got %s", k, describe(*v).c_str());
        *out = (uint32_t)v->num;
        return ok();
    };
    uint32_t nbits = 0, group = 0;
    TESSL_TRY(uint_key("bits", &nbits));
    TESSL_TRY(uint_key("group_size", &group));
    std::string mode = "affine";  // mlx-lm's own default when the key is absent
    if (const Json *m = q.get("mode")) {
        if (m->kind != Json::String) return fmt("config.json: quantization.mode: must be a string, got %s", describe(*m).c_str());
        mode = m->str;
    }
    if (mode != "affine") return fmt("config.json: quantization.mode is \"%s\"; only \"affine\" is supported", mode.c_str());
    if (nbits != kMlxQ4Bits) return fmt("config.json: quantization.bits is %u; only %u-bit weights are supported", nbits, kMlxQ4Bits);
    if (group != kMlxQ4Group)
        return fmt("config.json: quantization.group_size is %u; only %u is supported", group, kMlxQ4Group);
    *bits = nbits, *group_size = group;
    return ok();
}

std::string quoted_list(const std::vector<std::string> &v)
{
    std::string t = "[";
    for (size_t i = 0; i < v.size(); ++i) t += (i ? ", \"" : "\"") + v[i] + "\"";
    return t + "]";
}

bool starts_with(const char *s, const char *prefix) { return std::strncmp(s, prefix, std::strlen(prefix)) == 0; }

constexpr const char *kMlxPrefix = "language_model.model.", *kMlxHead = "language_model.lm_head";
constexpr const char *kHfPrefix = "model.language_model.", *kHfHead = "lm_head";

/// `MlxNames::detect` (src/qwen35_q4.rs:268-293): which spelling of the tower the names use; both is refused.
Result names_detect(const char *const *names, uint64_t n, const char **prefix, const char **head)
{
    bool mlx = false, hf = false;
    for (uint64_t i = 0; i < n; ++i) {
        if (!names[i]) return "MlxNames::detect: null name";
        mlx |= starts_with(names[i], kMlxPrefix);
        hf |= starts_with(names[i], kHfPrefix);
    }
    if (mlx && hf)
        return "checkpoint conventions: tensors under both \"language_model.model.\" and \"model.language_model.\"";
    if (!mlx && !hf)
        return "no tensor under \"language_model.model.\" (mlx-lm) or \"model.language_model.\" (Hugging Face): not a "
               "Qwen3.5 checkpoint";
    *prefix = mlx ? kMlxPrefix : kHfPrefix, *head = mlx ? kMlxHead : kHfHead;
    return ok();
}

/// `NormConvention::from_conv_shape` (src/qwen35_q4.rs:323-336): [conv_dim, 1, k] is the transformers layout (0),
/// [conv_dim, k, 1] the one `mlx_lm.convert` writes, whose zero-centred norms hold 1 + w (1).
Result norm_convention_from_conv_shape(const char *tensor, const uint64_t *shape, uint32_t ndim, uint64_t conv_dim,
                                       uint64_t kernel, uint32_t *convention)
{
    const std::vector<uint64_t> got(shape, shape + ndim), hf = {conv_dim, 1, kernel}, mlx = {conv_dim, kernel, 1};
    if (got == hf) return *convention = 0, ok();
    if (got == mlx) return *convention = 1, ok();
    return fmt("%s: shape %s, expected %s (4-bit packs eight values per U32 word; a different width means other bits)",
               tensor, shape_text(got).c_str(), shape_text(hf).c_str());
}

/// `classify_outside` (src/qwen35_q4.rs:350-373): tensors outside the tower that no read touched are either
/// skipped on purpose and by name - `mtp.*` (class 0), the vision tower (class 1) - or refused.
Result classify_outside(const char *const *names, uint64_t n, uint8_t *classes)
{
    static const char *kVision[4] = {"vision_tower.", "model.visual.", "visual.", "model.vision_tower."};
    std::vector<std::string> other;
    for (uint64_t i = 0; i < n; ++i) {
        if (!names[i]) return "classify_outside: null name";
        bool vision = false;
        for (const char *p : kVision) vision |= starts_with(names[i], p);
        if (starts_with(names[i], "mtp.")) {
            classes[i] = 0;
        } else if (vision) {
            classes[i] = 1;
        } else {
            classes[i] = 255;
            other.push_back(names[i]);
        }
    }
    if (other.empty()) return ok();
    const size_t count = other.size();
    if (other.size() > 8) other.resize(8);
    return fmt("%zu tensor(s) outside the tower that are neither its head nor mtp.* / the vision tower: %s", count,
               quoted_list(other).c_str());
}

void put_err(char *err, size_t err_len, const std::string &msg)
{
    if (!err || err_len == 0) return;
    size_t end = msg.size() < err_len - 1 ? msg.size() : err_len - 1;
    while (end > 0 && end < msg.size() && (static_cast<unsigned char>(msg[end]) & 0xC0) == 0x80) --end;
    std::memcpy(err, msg.data(), end);
    err[end] = 0;
}

template <typename F>
int32_t host_guarded(char *err, size_t err_len, F f)
{
    try {
        const Result r = f();
        if (r.empty()) return TESSL_OK;
        put_err(err, err_len, r);
        return TESSL_ERR;
    } catch (const std::exception &e) {
        put_err(err, err_len, std::string("panic in tessl: ") + e.what());
        return TESSL_PANIC;
    } catch (...) {
        put_err(err, err_len, "panic in tessl: unknown exception");
        return TESSL_PANIC;
    }
}

}  // namespace
}  // namespace tessl

using tessl::Result;

extern "C" {

TesslCheckpoint *tessl_checkpoint_open(const char *path, char *err, size_t err_len)
{
    std::unique_ptr<TesslCheckpoint> ck;
    const int32_t st = tessl::host_guarded(err, err_len, [&] { return tessl::open_checkpoint(path, &ck); });
    return st == TESSL_OK ? ck.release() : nullptr;
}

void tessl_checkpoint_close(TesslCheckpoint *ck) { delete ck; }

int32_t tessl_checkpoint_tensor_count(const TesslCheckpoint *ck, uint64_t *out, char *err, size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!ck || !out) return "tessl_checkpoint_tensor_count: null argument";
        *out = ck->names.size();
        return tessl::ok();
    });
}

int32_t tessl_checkpoint_tensor_name(const TesslCheckpoint *ck, uint64_t index, char *name, size_t name_len, char *err,
                                     size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!ck || !name || name_len == 0) return "tessl_checkpoint_tensor_name: null argument";
        if (index >= ck->names.size()) return tessl::fmt("tessl_checkpoint_tensor_name: index %llu of %zu", (unsigned long long)index, ck->names.size());
        const std::string &n = ck->names[index];
        if (n.size() + 1 > name_len) return tessl::fmt("tessl_checkpoint_tensor_name: the name needs %zu bytes", n.size() + 1);
        std::memcpy(name, n.c_str(), n.size() + 1);
        return tessl::ok();
    });
}

int32_t tessl_checkpoint_tensor_info(const TesslCheckpoint *ck, const char *name, TesslTensorInfo *out, char *err,
                                     size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!ck || !name || !out) return "tessl_checkpoint_tensor_info: null argument";
        const tessl::TensorEntry *e = nullptr;
        TESSL_TRY(tessl::find(*ck, name, &e));
        if (e->shape.size() > 8) return tessl::fmt("%s: %zu dimensions, at most 8 are reported", name, e->shape.size());
        std::memset(out, 0, sizeof *out);
        std::strncpy(out->dtype, e->dtype.c_str(), sizeof out->dtype - 1);
        out->ndim = (uint32_t)e->shape.size();
        for (size_t i = 0; i < e->shape.size(); ++i) out->shape[i] = e->shape[i];
        out->nbytes = e->end - e->begin;
        return tessl::ok();
    });
}

int32_t tessl_mlx_quant_from_config_json(const char *text, uint32_t *bits, uint32_t *group_size, char *err, size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!bits || !group_size) return "tessl_mlx_quant_from_config_json: null out";
        return tessl::quant_from_config_json(text, bits, group_size);
    });
}

int32_t tessl_mlx_names_detect(const char *const *names, uint64_t n, const char **prefix, const char **head, char *err,
                               size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if ((n && !names) || !prefix || !head) return "tessl_mlx_names_detect: null argument";
        return tessl::names_detect(names, n, prefix, head);
    });
}

int32_t tessl_mlx_norm_convention_from_conv_shape(const char *tensor, const uint64_t *shape, uint32_t ndim, uint64_t conv_dim,
                                                  uint64_t kernel, uint32_t *convention, char *err, size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!tensor || (ndim && !shape) || !convention) return "tessl_mlx_norm_convention_from_conv_shape: null argument";
        return tessl::norm_convention_from_conv_shape(tensor, shape, ndim, conv_dim, kernel, convention);
    });
}

int32_t tessl_mlx_classify_outside(const char *const *names, uint64_t n, uint8_t *classes, char *err, size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (n && (!names || !classes)) return "tessl_mlx_classify_outside: null argument";
        return tessl::classify_outside(names, n, classes);
    });
}

int32_t tessl_mlx_q4_check_part(const TesslCheckpoint *ck, const char *weight_name, uint64_t rows, uint64_t cols, char *err,
                                size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!ck || !weight_name) return "tessl_mlx_q4_check_part: null argument";
        return tessl::check_part(*ck, weight_name, rows, cols);
    });
}

int32_t tessl_mlx_q4_read_bank(const TesslCheckpoint *ck, const char *const *weight_names, const uint64_t *rows,
                               uint32_t nparts, uint64_t cols, void *packed, uint64_t packed_bytes, void *scales_biases,
                               uint64_t scales_biases_bytes, char *err, size_t err_len)
{
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!ck || !weight_names || !rows || !packed || !scales_biases) return "tessl_mlx_q4_read_bank: null argument";
        return tessl::read_bank(*ck, weight_names, rows, nparts, cols, static_cast<uint8_t *>(packed), packed_bytes,
                                static_cast<uint16_t *>(scales_biases), scales_biases_bytes);
    });
}

int32_t tessl_mlx_q4_load_bank(TesslRuntime *rt, const TesslCheckpoint *ck, const char *const *weight_names,
                               const uint64_t *rows, uint32_t nparts, uint64_t cols, TesslQ4MlxBank bank, char *err,
                               size_t err_len)
{
    if (!rt) {
        tessl::put_err(err, err_len, "null runtime handle");
        return TESSL_ERR;
    }
    if (std::this_thread::get_id() != rt->owner) {
        tessl::put_err(err, err_len, "tessl runtime used from a thread other than the one that created it");
        return TESSL_ERR;
    }
    if (rt->poisoned) {
        tessl::put_err(err, err_len, "the runtime is poisoned by an earlier GPU fault and must be recreated");
        return TESSL_ERR;
    }
    return tessl::host_guarded(err, err_len, [&]() -> Result {
        if (!ck || !weight_names || !rows) return "tessl_mlx_q4_load_bank: null argument";
        uint64_t total = 0;
        for (uint32_t i = 0; i < nparts; ++i) total += rows[i];
        // headers first: a hostile config over a tiny file is refused before anything is staged
        for (uint32_t i = 0; i < nparts; ++i) {
            if (!weight_names[i]) return "mlx_q4: null part name";
            TESSL_TRY(tessl::check_part(*ck, weight_names[i], rows[i], cols));
        }
        const uint64_t pbytes = total * (cols / 2), sbytes = total * (cols / tessl::kMlxQ4Group) * 4;
        TESSL_TRY(tessl::require(bank.packed, pbytes, 1, "mlx_q4 bank packed"));
        TESSL_TRY(tessl::require(bank.scales_biases, sbytes, 1, "mlx_q4 bank scales_biases"));
        std::vector<uint8_t> hp(pbytes);
        std::vector<uint16_t> hs(sbytes / 2);
        TESSL_TRY(tessl::read_bank(*ck, weight_names, rows, nparts, cols, hp.data(), pbytes, hs.data(), sbytes));
        cudaSetDevice(rt->device);
        TESSL_TRY(tessl::cuda_check(rt, cudaMemcpyAsync(bank.packed.ptr, hp.data(), pbytes, cudaMemcpyHostToDevice, rt->stream),
                                    "mlx_q4 upload"));
        TESSL_TRY(tessl::cuda_check(rt, cudaMemcpyAsync(bank.scales_biases.ptr, hs.data(), sbytes, cudaMemcpyHostToDevice, rt->stream),
                                    "mlx_q4 upload"));
        // the staging vectors die with this call: wait for the copies whatever the runtime's mode
        return tessl::cuda_check(rt, cudaStreamSynchronize(rt->stream), "mlx_q4 upload");
    });
}

}  // extern "C"
