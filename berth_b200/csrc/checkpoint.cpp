// EXL3 checkpoint reader (host only): safetensors shard headers, the sharded index, grouping of tensors into
// quantized linears, bitrate and codebook of each linear, packed sign unpacking, byte reads of single tensors.
// Mirrors berth's loader crate: crates/berth-exl3/src/safetensors.rs (shard header, span and bounds checks),
// checkpoint.rs:60-208 (single file or weight_map index, total_size check, shard paths confined to the
// directory), linear.rs:157-324 (grouping by the `.trellis` suffix, scale selection, codebook markers,
// bitrate from the trellis' last dimension), signs.rs:25-45 (bit i of a word = element i, set = -1.0).
// config.json is not read here: the kernels need shapes and bitrates, which the tensors carry.
#include "../../include/berth_b200_checkpoint.h"

#include <sys/stat.h>

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

constexpr uint64_t kMaxHeaderBytes = 64ull << 20;        // safetensors.rs:11
constexpr uint64_t kMaxPackedSignBytes = 64ull << 20;    // linear.rs:10
constexpr uint64_t kMaxIndexBytes = 256ull << 20;

struct BadField : std::runtime_error {
    BadField(const std::string& field, const std::string& what) : std::runtime_error("`" + field + "`: " + what) {}
};

// ---------------------------------------------------------------- a small JSON reader
// Enough for safetensors headers and the index file: objects (key order kept), arrays, strings with the
// standard escapes, numbers, true / false / null.
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0;
    bool is_u64 = false;
    bool fraction = false;   // the token was written with a fraction or an exponent
    uint64_t u64 = 0;
    std::string str;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* get(const std::string& key) const
    {
        for (const auto& m : members)
            if (m.first == key) return &m.second;
        return nullptr;
    }
    const char* kind_name() const
    {
        switch (kind) {
            case Null: return "null";
            case Bool: return "a boolean";
            case Number: return "a number";
            case String: return "a string";
            case Array: return "an array";
            default: return "an object";
        }
    }
};

class JsonParser {
public:
    JsonParser(const char* p, size_t n, const std::string& where) : p_(p), end_(p + n), where_(where) {}
    Json parse()
    {
        Json v = value(0);
        ws();
        if (p_ != end_) fail("trailing characters after the JSON value");
        return v;
    }

private:
    const char* p_;
    const char* end_;
    std::string where_;

    [[noreturn]] void fail(const std::string& what) const { throw BadField(where_, "JSON: " + what); }
    void ws()
    {
        while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
    }
    bool lit(const char* s)
    {
        const size_t n = std::strlen(s);
        if (size_t(end_ - p_) >= n && std::memcmp(p_, s, n) == 0) { p_ += n; return true; }
        return false;
    }
    static void utf8(std::string& out, unsigned cp)
    {
        if (cp < 0x80) out += char(cp);
        else if (cp < 0x800) { out += char(0xC0 | (cp >> 6)); out += char(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) { out += char(0xE0 | (cp >> 12)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
        else { out += char(0xF0 | (cp >> 18)); out += char(0x80 | ((cp >> 12) & 0x3F)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
    }
    unsigned hex4()
    {
        if (end_ - p_ < 4) fail("short \\u escape");
        unsigned v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = *p_++;
            v <<= 4;
            if (c >= '0' && c <= '9') v |= unsigned(c - '0');
            else if (c >= 'a' && c <= 'f') v |= unsigned(c - 'a' + 10);
            else if (c >= 'A' && c <= 'F') v |= unsigned(c - 'A' + 10);
            else fail("bad \\u escape");
        }
        return v;
    }
    std::string string()
    {
        if (p_ >= end_ || *p_ != '"') fail("expected a string");
        ++p_;
        std::string out;
        while (true) {
            if (p_ >= end_) fail("unterminated string");
            const char c = *p_++;
            if (c == '"') return out;
            if (c != '\\') { out += c; continue; }
            if (p_ >= end_) fail("unterminated escape");
            const char e = *p_++;
            switch (e) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp = hex4();
                    if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
                        p_ += 2;
                        const unsigned lo = hex4();
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: fail("unknown escape");
            }
        }
    }
    Json number()
    {
        const char* s = p_;
        bool integral = true;
        if (p_ < end_ && *p_ == '-') { ++p_; integral = false; }
        while (p_ < end_ && ((*p_ >= '0' && *p_ <= '9') || *p_ == '.' || *p_ == 'e' || *p_ == 'E' || *p_ == '+' || *p_ == '-')) {
            if (*p_ < '0' || *p_ > '9') integral = false;
            ++p_;
        }
        if (p_ == s) fail("expected a value");
        Json v;
        v.kind = Json::Number;
        const std::string text(s, p_);
        v.num = std::strtod(text.c_str(), nullptr);
        v.fraction = text.find_first_of(".eE") != std::string::npos;
        if (integral && text.size() <= 20) {
            unsigned long long u = 0;
            bool ok = true;
            for (char c : text) {
                const unsigned d = unsigned(c - '0');
                if (u > (0xffffffffffffffffull - d) / 10) { ok = false; break; }
                u = u * 10 + d;
            }
            v.is_u64 = ok;
            v.u64 = u;
        }
        return v;
    }
    Json value(int depth)
    {
        if (depth > 64) fail("nesting too deep");
        ws();
        if (p_ >= end_) fail("unexpected end");
        Json v;
        if (*p_ == '{') {
            ++p_;
            v.kind = Json::Object;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return v; }
            while (true) {
                ws();
                std::string key = string();
                ws();
                if (p_ >= end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                v.members.emplace_back(std::move(key), value(depth + 1));
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return v; }
                fail("expected ',' or '}'");
            }
        }
        if (*p_ == '[') {
            ++p_;
            v.kind = Json::Array;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return v; }
            while (true) {
                v.items.push_back(value(depth + 1));
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return v; }
                fail("expected ',' or ']'");
            }
        }
        if (*p_ == '"') { v.kind = Json::String; v.str = string(); return v; }
        if (lit("true")) { v.kind = Json::Bool; v.b = true; return v; }
        if (lit("false")) { v.kind = Json::Bool; return v; }
        if (lit("null")) return v;
        return number();
    }
};

// ---------------------------------------------------------------- tensors and shards
struct Tensor {
    std::string name, shard;
    int dtype = 0;
    std::vector<uint64_t> shape;
    uint64_t offset = 0, length = 0;
};

const char* const kDtypeNames[] = {"BOOL", "U8", "I8", "I16", "U16", "I32", "U32", "I64", "U64", "F16", "BF16", "F32", "F64",
                                   "F8_E4M3", "F8_E5M2", "F8_E8M0"};
const uint64_t kDtypeSizes[] = {1, 1, 1, 2, 2, 4, 4, 8, 8, 2, 2, 4, 8, 1, 1, 1};

int parse_dtype(const std::string& tensor, const std::string& name)
{
    for (int i = 0; i < 16; ++i)
        if (name == kDtypeNames[i]) return i;
    throw BadField(tensor + ".dtype", "unknown safetensors dtype `" + name + "`");
}

uint64_t expect_u64(const std::string& field, const Json& v)
{
    if (v.kind != Json::Number || !v.is_u64) throw BadField(field, std::string("expected an integer, got ") + v.kind_name());
    return v.u64;
}

bool mul_overflows(uint64_t a, uint64_t b, uint64_t& out)
{
    return __builtin_mul_overflow(a, b, &out);
}

struct File {
    std::FILE* f = nullptr;
    explicit File(const std::string& path) : f(std::fopen(path.c_str(), "rb"))
    {
        if (!f) throw BadField(path, std::string("cannot open: ") + std::strerror(errno));
    }
    ~File() { if (f) std::fclose(f); }
    File(const File&) = delete;
    File& operator=(const File&) = delete;
    void read_at(uint64_t off, void* dst, uint64_t n, const std::string& path)
    {
        if (fseeko(f, off_t(off), SEEK_SET) != 0) throw BadField(path, "seek failed");
        if (n && std::fread(dst, 1, n, f) != n) throw BadField(path, "short read");
    }
};

uint64_t file_size(const std::string& path)
{
    struct stat st;
    if (stat(path.c_str(), &st) != 0) throw BadField(path, std::string("cannot stat: ") + std::strerror(errno));
    return uint64_t(st.st_size);
}
bool is_file(const std::string& path)
{
    struct stat st;
    return stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}
bool is_dir(const std::string& path)
{
    struct stat st;
    return stat(path.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

std::string read_whole(const std::string& path, uint64_t limit)
{
    const uint64_t n = file_size(path);
    if (n > limit) throw BadField(path, "file of " + std::to_string(n) + " bytes is too large");
    std::string s(n, '\0');
    File f(path);
    f.read_at(0, s.data(), n, path);
    return s;
}

// One tensor entry of a shard header (safetensors.rs:144-208): dtype, shape, data_offsets; the span must
// equal the shape's byte length and end inside the file.
Tensor parse_tensor(const std::string& path, const std::string& name, const Json& entry, uint64_t data_start, uint64_t file_len)
{
    if (entry.kind != Json::Object) throw BadField(name, std::string("expected a tensor object, got ") + entry.kind_name());
    const Json* dt = entry.get("dtype");
    if (!dt) throw BadField(name + ".dtype", "missing dtype");
    if (dt->kind != Json::String) throw BadField(name + ".dtype", "expected a string");
    Tensor t;
    t.name = name;
    t.shard = path;
    t.dtype = parse_dtype(name, dt->str);
    const Json* sh = entry.get("shape");
    if (!sh) throw BadField(name + ".shape", "missing shape");
    if (sh->kind != Json::Array) throw BadField(name + ".shape", std::string("expected an array, got ") + sh->kind_name());
    for (const Json& d : sh->items) t.shape.push_back(expect_u64(name + ".shape", d));
    if (t.shape.size() > 8) throw BadField(name + ".shape", "rank above 8");
    const Json* off = entry.get("data_offsets");
    if (!off) throw BadField(name + ".data_offsets", "missing data_offsets");
    if (off->kind != Json::Array) throw BadField(name + ".data_offsets", std::string("expected an array, got ") + off->kind_name());
    if (off->items.size() != 2) throw BadField(name + ".data_offsets", "expected 2 offsets, got " + std::to_string(off->items.size()));
    const uint64_t start = expect_u64(name + ".data_offsets", off->items[0]), end = expect_u64(name + ".data_offsets", off->items[1]);
    if (end < start) throw BadField(name + ".data_offsets", "end " + std::to_string(end) + " is before start " + std::to_string(start));
    const uint64_t span = end - start;
    uint64_t numel = 1;
    for (uint64_t d : t.shape)
        if (mul_overflows(numel, d, numel)) throw BadField(name, "shape product overflows u64");
    uint64_t nbytes;
    if (mul_overflows(numel, kDtypeSizes[t.dtype], nbytes)) throw BadField(name, "byte length overflows u64");
    if (span != nbytes)
        throw BadField(name, "data_offsets span " + std::to_string(span) + " does not match " + kDtypeNames[t.dtype] + " shape byte length " +
                                 std::to_string(nbytes));
    if (__builtin_add_overflow(data_start, start, &t.offset)) throw BadField(name, "byte offset overflows u64");
    uint64_t end_abs;
    if (__builtin_add_overflow(t.offset, span, &end_abs)) throw BadField(name, "tensor end overflows u64");
    if (end_abs > file_len)
        throw BadField(name, "tensor extends to byte " + std::to_string(end_abs) + " but the shard is " + std::to_string(file_len) + " bytes");
    t.length = span;
    return t;
}

// All tensors of one shard file (safetensors.rs:85-142): 8-byte little-endian header length, JSON header.
std::vector<Tensor> read_shard(const std::string& path)
{
    const uint64_t file_len = file_size(path);
    File f(path);
    unsigned char lenb[8];
    if (file_len < 8) throw BadField(path, "file is shorter than a safetensors header length");
    f.read_at(0, lenb, 8, path);
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | lenb[i];
    if (header_len > kMaxHeaderBytes || header_len > file_len - 8)
        throw BadField(path, "safetensors header length " + std::to_string(header_len) + " is not usable in a " + std::to_string(file_len) +
                                 "-byte file");
    std::string header(header_len, '\0');
    f.read_at(8, header.data(), header_len, path);
    const Json root = JsonParser(header.data(), header.size(), path).parse();
    if (root.kind != Json::Object) throw BadField(path, "safetensors header is not a JSON object");
    std::vector<Tensor> out;
    std::set<std::string> seen;
    for (const auto& m : root.members) {
        if (m.first == "__metadata__") continue;
        if (!seen.insert(m.first).second) throw BadField(m.first, "duplicated inside one shard header");
        out.push_back(parse_tensor(path, m.first, m.second, 8 + header_len, file_len));
    }
    return out;
}

using Index = std::map<std::string, Tensor>;   // name order, as berth's BTreeMap

void insert_tensor(Index& index, Tensor t)
{
    const std::string name = t.name;
    if (!index.emplace(name, std::move(t)).second) throw BadField(name, "tensor name appears more than once");
}

// A shard named by the index must stay inside the checkpoint directory (checkpoint.rs:193-208).
std::string shard_path(const std::string& dir, const std::string& rel)
{
    bool escapes = !rel.empty() && rel[0] == '/';
    size_t i = 0;
    while (i <= rel.size()) {
        const size_t j = rel.find('/', i);
        const std::string comp = rel.substr(i, j == std::string::npos ? std::string::npos : j - i);
        if (comp == "..") escapes = true;
        if (j == std::string::npos) break;
        i = j + 1;
    }
    if (escapes) throw BadField("weight_map", "shard `" + rel + "` is not a path inside the checkpoint directory");
    return dir + "/" + rel;
}

// The directory's tensors and the index file's metadata.total_size, if it has one (checkpoint.rs:87-190).
Index read_tensors(const std::string& dir, bool& has_total, uint64_t& total_size)
{
    has_total = false;
    Index index;
    const std::string index_path = dir + "/model.safetensors.index.json";
    if (is_file(index_path)) {
        const std::string text = read_whole(index_path, kMaxIndexBytes);
        const Json root = JsonParser(text.data(), text.size(), "model.safetensors.index.json").parse();
        if (root.kind != Json::Object) throw BadField("model.safetensors.index.json", "expected a JSON object");
        const Json* wm = root.get("weight_map");
        if (!wm) throw BadField("weight_map", "missing field");
        if (wm->kind != Json::Object) throw BadField("weight_map", "expected an object");
        std::map<std::string, std::set<std::string>> by_shard;
        for (const auto& m : wm->members) {
            if (m.second.kind != Json::String) throw BadField("weight_map." + m.first, "expected a shard filename");
            if (m.second.str.empty()) throw BadField("weight_map." + m.first, "empty shard path");
            by_shard[shard_path(dir, m.second.str)].insert(m.first);
        }
        if (const Json* meta = root.get("metadata")) {
            if (meta->kind != Json::Object) throw BadField("metadata", "expected an object");
            if (const Json* ts = meta->get("total_size")) {
                if (ts->kind != Json::Number || !ts->is_u64) throw BadField("metadata.total_size", "expected an integer");
                has_total = true;
                total_size = ts->u64;
            }
        }
        for (const auto& [path, expected] : by_shard) {
            std::set<std::string> saw;
            for (Tensor& t : read_shard(path)) {
                if (!expected.count(t.name)) throw BadField(t.name, "present in " + path + " but not in model.safetensors.index.json");
                saw.insert(t.name);
                insert_tensor(index, std::move(t));
            }
            for (const std::string& name : expected)
                if (!saw.count(name)) throw BadField(name, "weight_map lists it in " + path + " but the shard header does not");
        }
        return index;
    }
    const std::string single = dir + "/model.safetensors";
    if (is_file(single)) {
        for (Tensor& t : read_shard(single)) insert_tensor(index, std::move(t));
        return index;
    }
    throw BadField("model.safetensors", "no model.safetensors.index.json and no model.safetensors");
}

// ---------------------------------------------------------------- linears
struct Linear {
    std::string prefix;
    Tensor trellis, input_scale, output_scale, bias;
    bool input_packed = false, output_packed = false, has_bias = false;
    int codebook = 0;   // 0 default, 1 mcg, 2 mul1
    int bits_x2 = 0;
};

const char* const kLinearParts[] = {"trellis", "suh", "svh", "su", "sv", "bias", "mcg", "mul1"};   // linear.rs:12

const Tensor* find(const Index& index, const std::string& name)
{
    const auto it = index.find(name);
    return it == index.end() ? nullptr : &it->second;
}

// Last dimension of the trellis = 16 * K words, or 16 * floor(K) + 8 for the half rates 1.5 / 2.5 / 3.5, which
// exist only with the mul1 codebook (linear.rs:285-324).
int bitrate_x2(const std::string& tensor, uint64_t last, int codebook)
{
    if (last % 16 == 0) {
        const uint64_t k = last / 16;
        if (k >= 1 && k <= 8) return int(2 * k);
        throw BadField(tensor, "integer bitrate " + std::to_string(k) + " is outside 1..=8 (last dim " + std::to_string(last) + ")");
    }
    if (last % 16 == 8) {
        const uint64_t fl = last / 16;
        if (fl < 1 || fl > 3)
            throw BadField(tensor, "half-integer bitrate " + std::to_string(fl) + ".5 is not one of 1.5, 2.5, 3.5 (last dim " +
                                       std::to_string(last) + ")");
        if (codebook != 2)
            throw BadField(tensor, "half-integer bitrate " + std::to_string(fl) + ".5 requires mul1 (last dim " + std::to_string(last) + ")");
        return int(2 * fl + 1);
    }
    throw BadField(tensor, "last dim " + std::to_string(last) + " is not 16*K or 16*K+8");
}

// The unpacked fp16 vector wins when both are stored (linear.rs:243-276).
Tensor pick_scale(const Index& index, const std::string& prefix, const char* unpacked_suffix, const char* packed_suffix, bool& packed)
{
    const Tensor* u = find(index, prefix + "." + unpacked_suffix);
    const Tensor* p = find(index, prefix + "." + packed_suffix);
    if (u && u->dtype != BERTH_DT_F16) throw BadField(u->name, std::string("expected F16, got ") + kDtypeNames[u->dtype]);
    if (p && p->dtype != BERTH_DT_I16) throw BadField(p->name, std::string("expected I16, got ") + kDtypeNames[p->dtype]);
    if (u) { packed = false; return *u; }
    if (p) { packed = true; return *p; }
    throw BadField(prefix + "." + unpacked_suffix, std::string("missing ") + unpacked_suffix + " or " + packed_suffix);
}

Linear build_linear(const Index& index, const std::string& prefix)
{
    Linear l;
    l.prefix = prefix;
    const Tensor* t = find(index, prefix + ".trellis");
    if (!t) throw BadField(prefix + ".trellis", "missing trellis");
    if (t->dtype != BERTH_DT_I16) throw BadField(t->name, std::string("expected I16, got ") + kDtypeNames[t->dtype]);
    if (t->shape.size() != 3) throw BadField(t->name, "expected rank 3, got rank " + std::to_string(t->shape.size()));
    l.trellis = *t;
    const bool mcg = find(index, prefix + ".mcg"), mul1 = find(index, prefix + ".mul1");
    if (mcg && mul1) throw BadField(prefix + ".mcg", "both mcg and mul1 are present");
    l.codebook = mul1 ? 2 : (mcg ? 1 : 0);
    l.bits_x2 = bitrate_x2(t->name, t->shape[2], l.codebook);
    l.input_scale = pick_scale(index, prefix, "suh", "su", l.input_packed);
    l.output_scale = pick_scale(index, prefix, "svh", "sv", l.output_packed);
    if (const Tensor* b = find(index, prefix + ".bias")) {
        if (b->dtype != BERTH_DT_F16 && b->dtype != BERTH_DT_BF16 && b->dtype != BERTH_DT_F32)
            throw BadField(b->name, std::string("expected a float bias, got ") + kDtypeNames[b->dtype]);
        l.bias = *b;
        l.has_bias = true;
    }
    return l;
}

}  // namespace

struct berth_ckpt {
    std::string directory;
    Index tensors;
    std::vector<const Tensor*> by_order;   // name order
    std::vector<Linear> linears;           // prefix order
    std::vector<const Tensor*> others;     // tensors no linear consumed, name order
};

namespace {

thread_local std::string g_error;

template <typename F>
int guarded(F&& f)
{
    try {
        g_error.clear();
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
    } catch (...) {
        g_error = "unknown error";
    }
    return -1;
}

void fill(const Tensor& t, berth_tensor_info* out)
{
    std::memset(out, 0, sizeof(*out));
    out->name = t.name.c_str();
    out->shard = t.shard.c_str();
    out->dtype = t.dtype;
    out->rank = int(t.shape.size());
    for (size_t i = 0; i < t.shape.size(); ++i) out->shape[i] = t.shape[i];
    out->offset = t.offset;
    out->length = t.length;
}

void fill(const Linear& l, berth_linear_info* out)
{
    std::memset(out, 0, sizeof(*out));
    out->prefix = l.prefix.c_str();
    fill(l.trellis, &out->trellis);
    fill(l.input_scale, &out->input_scale);
    fill(l.output_scale, &out->output_scale);
    if (l.has_bias) fill(l.bias, &out->bias);
    out->input_packed = l.input_packed;
    out->output_packed = l.output_packed;
    out->has_bias = l.has_bias;
    out->codebook = l.codebook;
    out->bits_x2 = l.bits_x2;
}

void need(const void* p, const char* what)
{
    if (!p) throw std::runtime_error(std::string("checkpoint: null ") + what);
}

void read_tensor(const Tensor& t, void* dst)
{
    File f(t.shard);
    f.read_at(t.offset, dst, t.length, t.shard);
}

void unpack_signs(const unsigned char* packed, uint64_t bytes, uint16_t* out)
{
    if (bytes % 2 != 0) throw BadField("su", "packed sign bytes " + std::to_string(bytes) + " are not a multiple of 2");
    for (uint64_t w = 0; w < bytes / 2; ++w) {
        const unsigned word = unsigned(packed[2 * w]) | (unsigned(packed[2 * w + 1]) << 8);
        for (int bit = 0; bit < 16; ++bit) out[w * 16 + bit] = ((word >> bit) & 1u) ? 0xBC00 : 0x3C00;
    }
}

const Linear& linear_named(const berth_ckpt* c, const char* prefix)
{
    // (prefix order: binary search)
    size_t lo = 0, hi = c->linears.size();
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (c->linears[mid].prefix < prefix) lo = mid + 1; else hi = mid;
    }
    if (lo == c->linears.size() || c->linears[lo].prefix != prefix) throw BadField(prefix, "no such linear");
    return c->linears[lo];
}

}  // namespace

extern "C" const char* berth_ckpt_last_error(void) { return g_error.c_str(); }

extern "C" int berth_ckpt_open(const char* directory, berth_ckpt** out)
{
    return guarded([&] {
        need(directory, "directory");
        need(out, "output handle");
        *out = nullptr;
        if (!is_dir(directory)) throw BadField(directory, "not a checkpoint directory");
        auto c = std::make_unique<berth_ckpt>();
        c->directory = directory;
        bool has_total = false;
        uint64_t total = 0;
        c->tensors = read_tensors(c->directory, has_total, total);
        if (has_total) {
            uint64_t sum = 0;
            for (const auto& kv : c->tensors)
                if (__builtin_add_overflow(sum, kv.second.length, &sum)) throw BadField("metadata.total_size", "tensor byte sum overflows u64");
            if (sum != total)
                throw BadField("metadata.total_size", "index says " + std::to_string(total) + ", tensor bytes sum to " + std::to_string(sum));
        }
        // group_linears (linear.rs:157-185): every `<prefix>.trellis` makes a linear that consumes its sibling parts
        std::set<std::string> consumed;
        for (const auto& kv : c->tensors) {
            c->by_order.push_back(&kv.second);
            const std::string& name = kv.first;
            const std::string suffix = ".trellis";
            if (name.size() < suffix.size() || name.compare(name.size() - suffix.size(), suffix.size(), suffix) != 0) continue;
            const std::string prefix = name.substr(0, name.size() - suffix.size());
            if (prefix.empty()) throw BadField(name, "trellis tensor has an empty linear prefix");
            c->linears.push_back(build_linear(c->tensors, prefix));
            for (const char* part : kLinearParts)
                if (c->tensors.count(prefix + "." + part)) consumed.insert(prefix + "." + part);
        }
        std::sort(c->linears.begin(), c->linears.end(), [](const Linear& a, const Linear& b) { return a.prefix < b.prefix; });
        for (const auto& kv : c->tensors)
            if (!consumed.count(kv.first)) c->others.push_back(&kv.second);
        *out = c.release();
    });
}

extern "C" void berth_ckpt_close(berth_ckpt* ckpt) { delete ckpt; }

extern "C" int64_t berth_ckpt_n_tensors(const berth_ckpt* c) { return c ? int64_t(c->by_order.size()) : -1; }
extern "C" int64_t berth_ckpt_n_linears(const berth_ckpt* c) { return c ? int64_t(c->linears.size()) : -1; }
extern "C" int64_t berth_ckpt_n_others(const berth_ckpt* c) { return c ? int64_t(c->others.size()) : -1; }

extern "C" int berth_ckpt_tensor_at(const berth_ckpt* c, int64_t i, berth_tensor_info* out)
{
    return guarded([&] {
        need(c, "checkpoint"); need(out, "output");
        if (i < 0 || i >= int64_t(c->by_order.size())) throw std::runtime_error("checkpoint: tensor index out of range");
        fill(*c->by_order[size_t(i)], out);
    });
}

extern "C" int berth_ckpt_tensor(const berth_ckpt* c, const char* name, berth_tensor_info* out)
{
    return guarded([&] {
        need(c, "checkpoint"); need(name, "name"); need(out, "output");
        const Tensor* t = find(c->tensors, name);
        if (!t) throw BadField(name, "no such tensor");
        fill(*t, out);
    });
}

extern "C" int berth_ckpt_linear_at(const berth_ckpt* c, int64_t i, berth_linear_info* out)
{
    return guarded([&] {
        need(c, "checkpoint"); need(out, "output");
        if (i < 0 || i >= int64_t(c->linears.size())) throw std::runtime_error("checkpoint: linear index out of range");
        fill(c->linears[size_t(i)], out);
    });
}

extern "C" int berth_ckpt_linear(const berth_ckpt* c, const char* prefix, berth_linear_info* out)
{
    return guarded([&] {
        need(c, "checkpoint"); need(prefix, "prefix"); need(out, "output");
        fill(linear_named(c, prefix), out);
    });
}

extern "C" int berth_ckpt_other_at(const berth_ckpt* c, int64_t i, berth_tensor_info* out)
{
    return guarded([&] {
        need(c, "checkpoint"); need(out, "output");
        if (i < 0 || i >= int64_t(c->others.size())) throw std::runtime_error("checkpoint: tensor index out of range");
        fill(*c->others[size_t(i)], out);
    });
}

extern "C" int berth_ckpt_read(const berth_ckpt* c, const char* name, void* dst, uint64_t dst_bytes)
{
    return guarded([&] {
        need(c, "checkpoint"); need(name, "name"); need(dst, "destination");
        const Tensor* t = find(c->tensors, name);
        if (!t) throw BadField(name, "no such tensor");
        if (dst_bytes != t->length)
            throw BadField(name, "destination of " + std::to_string(dst_bytes) + " bytes, tensor of " + std::to_string(t->length));
        read_tensor(*t, dst);
    });
}

extern "C" int berth_ckpt_scale_f16(const berth_ckpt* c, const char* prefix, int output_side, uint16_t* dst, uint64_t dst_halves)
{
    return guarded([&] {
        need(c, "checkpoint"); need(prefix, "prefix"); need(dst, "destination");
        const Linear& l = linear_named(c, prefix);
        const Tensor& t = output_side ? l.output_scale : l.input_scale;
        const bool packed = output_side ? l.output_packed : l.input_packed;
        const uint64_t channels = packed ? t.length * 8 : t.length / 2;
        if (dst_halves != channels)
            throw BadField(t.name, "destination of " + std::to_string(dst_halves) + " values, scale of " + std::to_string(channels));
        if (!packed) { read_tensor(t, dst); return; }
        if (t.length > kMaxPackedSignBytes)
            throw BadField(t.name, "refusing to read " + std::to_string(t.length) + " bytes; packed sign reads are capped at " +
                                       std::to_string(kMaxPackedSignBytes));
        std::vector<unsigned char> bytes(t.length);
        read_tensor(t, bytes.data());
        unpack_signs(bytes.data(), t.length, dst);
    });
}

extern "C" int berth_unpack_signs(const void* packed_le, uint64_t bytes, uint16_t* out)
{
    return guarded([&] {
        if (bytes) { need(packed_le, "packed signs"); need(out, "output"); }
        unpack_signs(static_cast<const unsigned char*>(packed_le), bytes, out);
    });
}

// ---------------------------------------------------------------- config.json (crates/berth-exl3/src/config.rs)
namespace {

struct MissingField : std::runtime_error {
    explicit MissingField(const std::string& field) : std::runtime_error("missing field `" + field + "`") {}
};
struct BadConfig : std::runtime_error {
    BadConfig(const std::string& field, const std::string& detail) : std::runtime_error("field `" + field + "`: " + detail) {}
};

// A number as serde_json prints it: integers without a fraction, other values with the shortest digits that read back.
std::string number_text(const Json& v)
{
    if (v.is_u64) return std::to_string(v.u64);
    if (std::isfinite(v.num) && v.num == std::floor(v.num) && std::fabs(v.num) < 9.0e15 && !v.fraction)
        return std::to_string((long long) v.num);
    char buf[40];
    for (int prec = 1; prec <= 17; ++prec) {
        std::snprintf(buf, sizeof buf, "%.*g", prec, v.num);
        if (std::strtod(buf, nullptr) == v.num) break;
    }
    std::string s(buf);
    if (s.find_first_of(".eEn") == std::string::npos) s += ".0";
    return s;
}
std::string quoted(const std::string& s)
{
    std::string out = "\"";
    for (char c : s) {
        if (c == '"' || c == '\\') { out += '\\'; out += c; }
        else if (c == '\n') out += "\\n";
        else if (c == '\t') out += "\\t";
        else if (c == '\r') out += "\\r";
        else out += c;
    }
    return out + "\"";
}
// config.rs:381-391
std::string describe(const Json& v)
{
    switch (v.kind) {
        case Json::Null: return "null";
        case Json::Bool: return v.b ? "true" : "false";
        case Json::Number: return number_text(v);
        case Json::String: return v.str.size() < 64 ? "string " + quoted(v.str) : "a long string";
        case Json::Array: return "an array";
        default: return "an object";
    }
}
const Json* lookup(const Json& root, const Json* text, const char* key)
{
    if (text)
        if (const Json* v = text->get(key)) return v;
    return root.get(key);
}
const Json& require(const Json& root, const Json* text, const char* key)
{
    const Json* v = lookup(root, text, key);
    if (!v) throw MissingField(key);
    return *v;
}
// Integers, or floats that are exactly an integer (config.rs:360-379).
uint32_t expect_u32(const Json& v, const std::string& field)
{
    if (v.kind == Json::Number) {
        if (v.is_u64) {
            if (v.u64 > 0xffffffffull) throw BadConfig(field, "integer " + std::to_string(v.u64) + " does not fit in u32");
            return uint32_t(v.u64);
        }
        if (std::isfinite(v.num) && v.num >= 0.0 && v.num == std::floor(v.num) && v.num <= 4294967295.0) return uint32_t(v.num);
    }
    throw BadConfig(field, "expected a non-negative integer, got " + describe(v));
}
bool expect_bool(const Json& v, const std::string& field)
{
    if (v.kind != Json::Bool) throw BadConfig(field, "expected a bool, got " + describe(v));
    return v.b;
}
std::string expect_string(const Json& v, const std::string& field)
{
    if (v.kind != Json::String) throw BadConfig(field, "expected a string, got " + describe(v));
    return v.str;
}

}  // namespace

struct berth_config_strings {
    std::string arch, quant_method, codebook, version, out_scales;
    std::vector<std::string> layer_types;
    std::vector<const char*> layer_ptrs;
};

namespace {

void parse_config(const char* json, uint64_t bytes, berth_model_config& c, berth_config_strings& s)
{
    const Json root = JsonParser(json, size_t(bytes), "config.json").parse();
    if (root.kind != Json::Object) throw BadConfig("config.json", "expected a JSON object");
    const Json* text = root.get("text_config");
    if (text && text->kind != Json::Object) throw BadConfig("text_config", "expected an object, got " + describe(*text));

    const Json* arch = root.get("architectures");
    if (!arch) throw MissingField("architectures");
    if (arch->kind != Json::Array) throw BadConfig("architectures", "expected an array, got " + describe(*arch));
    if (arch->items.empty()) throw BadConfig("architectures", "expected a non-empty array");
    if (arch->items[0].kind != Json::String) throw BadConfig("architectures", "expected a string, got " + describe(arch->items[0]));
    if (arch->items[0].str.empty()) throw BadConfig("architectures", "architecture string is empty");
    s.arch = arch->items[0].str;

    c.num_hidden_layers = expect_u32(require(root, text, "num_hidden_layers"), "num_hidden_layers");
    const Json& lt = require(root, text, "layer_types");
    if (lt.kind != Json::Array) throw BadConfig("layer_types", "expected an array, got " + describe(lt));
    for (const Json& item : lt.items) {
        if (item.kind != Json::String) throw BadConfig("layer_types", "expected strings, got " + describe(item));
        s.layer_types.push_back(item.str);
    }
    if (s.layer_types.size() != c.num_hidden_layers)
        throw BadConfig("layer_types", "length " + std::to_string(s.layer_types.size()) + " does not match num_hidden_layers " +
                                           std::to_string(c.num_hidden_layers));
    const Json* quant = root.get("quantization_config");
    if (!quant) throw MissingField("quantization_config");

    auto req = [&](const char* key) { return expect_u32(require(root, text, key), key); };
    auto opt = [&](const char* key) -> int64_t {
        const Json* v = lookup(root, text, key);
        return v ? int64_t(expect_u32(*v, key)) : -1;
    };
    c.hidden_size = req("hidden_size");
    c.intermediate_size = opt("intermediate_size");
    c.head_dim = req("head_dim");
    c.num_attention_heads = req("num_attention_heads");
    c.num_key_value_heads = req("num_key_value_heads");
    c.vocab_size = req("vocab_size");
    c.tie_word_embeddings = expect_bool(require(root, text, "tie_word_embeddings"), "tie_word_embeddings") ? 1 : 0;
    c.linear_conv_kernel_dim = req("linear_conv_kernel_dim");
    c.linear_num_key_heads = req("linear_num_key_heads");
    c.linear_num_value_heads = req("linear_num_value_heads");
    c.linear_key_head_dim = req("linear_key_head_dim");
    c.linear_value_head_dim = req("linear_value_head_dim");
    c.attn_output_gate = expect_bool(require(root, text, "attn_output_gate"), "attn_output_gate") ? 1 : 0;
    c.num_experts = opt("num_experts");
    c.num_experts_per_tok = opt("num_experts_per_tok");
    c.moe_intermediate_size = opt("moe_intermediate_size");
    c.shared_expert_intermediate_size = opt("shared_expert_intermediate_size");

    if (quant->kind != Json::Object) throw BadConfig("quantization_config", "expected an object, got " + describe(*quant));
    auto qreq = [&](const char* key) -> const Json& {
        const Json* v = quant->get(key);
        if (!v) throw MissingField(key);
        return *v;
    };
    c.calibration_rows = c.calibration_cols = -1;
    if (const Json* cal = quant->get("calibration")) {
        if (cal->kind != Json::Object) throw BadConfig("calibration", "expected an object, got " + describe(*cal));
        const Json* rows = cal->get("rows");
        if (!rows) throw MissingField("calibration.rows");
        const Json* cols = cal->get("cols");
        if (!cols) throw MissingField("calibration.cols");
        c.calibration_rows = expect_u32(*rows, "calibration.rows");
        c.calibration_cols = expect_u32(*cols, "calibration.cols");
    }
    s.quant_method = expect_string(qreq("quant_method"), "quant_method");
    const Json& bits = qreq("bits");
    if (bits.kind != Json::Number) throw BadConfig("bits", "expected a number, got " + describe(bits));
    if (!std::isfinite(bits.num) || bits.num < 0.0) throw BadConfig("bits", "expected a non-negative finite number, got " + number_text(bits));
    c.bits = bits.num;
    c.head_bits = expect_u32(qreq("head_bits"), "head_bits");
    auto qstr = [&](const char* key, std::string& dst) -> const char* {
        const Json* v = quant->get(key);
        if (!v) return nullptr;
        dst = expect_string(*v, key);
        return dst.c_str();
    };
    auto qopt = [&](const char* key) -> int64_t {
        const Json* v = quant->get(key);
        return v ? int64_t(expect_u32(*v, key)) : -1;
    };
    c.codebook = qstr("codebook", s.codebook);
    c.version = qstr("version", s.version);
    c.vision_bits = qopt("vision_bits");
    c.mtp_bits = qopt("mtp_bits");
    c.out_scales = qstr("out_scales", s.out_scales);
    c.arch_string = s.arch.c_str();
    c.quant_method = s.quant_method.c_str();
    for (const std::string& t : s.layer_types) s.layer_ptrs.push_back(t.c_str());
    c.n_layer_types = int64_t(s.layer_ptrs.size());
    c.layer_types = s.layer_ptrs.data();
}

}  // namespace

extern "C" int berth_config_parse(const char* json, uint64_t bytes, berth_model_config** out)
{
    return guarded([&] {
        need(json, "json");
        need(out, "out");
        *out = nullptr;
        auto* c = new berth_model_config();
        auto* s = new berth_config_strings();
        c->strings = s;
        try {
            parse_config(json, bytes, *c, *s);
        } catch (...) {
            delete s;
            delete c;
            throw;
        }
        *out = c;
    });
}

extern "C" int berth_config_open(const char* directory, berth_model_config** out)
{
    std::string text;
    const int rc = guarded([&] {
        need(directory, "directory");
        need(out, "out");
        *out = nullptr;
        const std::string path = std::string(directory) + "/config.json";
        if (!is_file(path)) throw std::runtime_error(path + ": No such file or directory");
        text = read_whole(path, kMaxIndexBytes);
    });
    if (rc != 0) return rc;
    return berth_config_parse(text.data(), text.size(), out);
}

extern "C" void berth_config_free(berth_model_config* c)
{
    if (!c) return;
    delete c->strings;
    delete c;
}
