// Bounded safetensors metadata ingestion (vyre-safetensors/src/lib.rs:16-260, 871-907): one shard's header is read and
// validated without touching tensor payloads - prefix, header size limit, JSON object of {dtype, shape, data_offsets},
// `__metadata__` ignored, duplicate names refused, every range inside the payload, byte length = shape x dtype width,
// no two ranges overlapping - and identified by the BLAKE3 of its exact header bytes, the file length and the payload
// start. Tensor bytes then go straight from the file into a resident device buffer (vyb_safetensors_upload).
// Sharded indexes (model.safetensors.index.json) and full-checkpoint content identities are not rebuilt.
#include <algorithm>
#include <cstdio>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "blake3.hpp"
#include "model.hpp"

namespace vyb {
namespace {

constexpr uint64_t MAX_HEADER_BYTES = 64ull * 1024 * 1024;  // lib.rs:16
constexpr size_t MAX_TENSORS = 1000000;                      // lib.rs:18
constexpr size_t MAX_TENSOR_NAME_BYTES = 4096;               // lib.rs:19

struct DtypeInfo {
    const char* name;
    uint32_t width;
};
// lib.rs:27-71; the order is the tag returned through the C ABI
const DtypeInfo DTYPES[] = {{"BOOL", 1}, {"U8", 1},  {"I8", 1},  {"U16", 2}, {"I16", 2}, {"U32", 4},     {"I32", 4},    {"U64", 8},
                            {"I64", 8},  {"F16", 2}, {"BF16", 2}, {"F32", 4}, {"F64", 8}, {"F8_E4M3", 1}, {"F8_E5M2", 1}};

struct Entry {
    std::string name;
    uint32_t dtype = 0;
    std::vector<uint64_t> shape;
    uint64_t begin = 0, end = 0;  // absolute byte range in the file
};

// ---- a JSON reader for exactly what a safetensors header holds ----------------------------------------------------------
struct Json {
    const uint8_t* p;
    const uint8_t* e;
    std::string err;
    bool fail(const std::string& m) {
        if (err.empty()) err = m + " at byte " + std::to_string(p_off());
        return false;
    }
    const uint8_t* base;
    size_t p_off() const { return size_t(p - base); }
    void ws() {
        while (p < e && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
    }
    bool eat(char c) {
        ws();
        if (p < e && *p == uint8_t(c)) {
            ++p;
            return true;
        }
        return false;
    }
    bool expect(char c) { return eat(c) || fail(std::string("expected `") + c + "`"); }
    bool string(std::string* out) {
        ws();
        if (p >= e || *p != '"') return fail("expected a string");
        ++p;
        out->clear();
        while (p < e && *p != '"') {
            if (*p < 0x20) return fail("control character in a string");
            if (*p == '\\') {
                if (++p >= e) return fail("unterminated escape");
                switch (*p) {
                    case '"': out->push_back('"'); break;
                    case '\\': out->push_back('\\'); break;
                    case '/': out->push_back('/'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'n': out->push_back('\n'); break;
                    case 'r': out->push_back('\r'); break;
                    case 't': out->push_back('\t'); break;
                    case 'u': {
                        if (e - p < 5) return fail("short \\u escape");
                        uint32_t cp = 0;
                        for (int i = 1; i <= 4; ++i) {
                            const uint8_t c = p[i];
                            cp = cp * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 0x10000);
                        }
                        if (cp > 0xFFFF) return fail("bad \\u escape");
                        p += 4;
                        if (cp >= 0xD800 && cp <= 0xDFFF) return fail("surrogate escapes are not accepted in tensor names");
                        if (cp < 0x80) {
                            out->push_back(char(cp));
                        } else if (cp < 0x800) {
                            out->push_back(char(0xC0 | (cp >> 6)));
                            out->push_back(char(0x80 | (cp & 0x3F)));
                        } else {
                            out->push_back(char(0xE0 | (cp >> 12)));
                            out->push_back(char(0x80 | ((cp >> 6) & 0x3F)));
                            out->push_back(char(0x80 | (cp & 0x3F)));
                        }
                        break;
                    }
                    default: return fail("unknown escape");
                }
                ++p;
            } else {
                out->push_back(char(*p++));
            }
        }
        if (p >= e) return fail("unterminated string");
        ++p;
        return true;
    }
    bool u64(uint64_t* out) {
        ws();
        if (p >= e || *p < '0' || *p > '9') return fail("expected an unsigned integer");
        uint64_t v = 0;
        while (p < e && *p >= '0' && *p <= '9') {
            const uint64_t d = *p - '0';
            if (v > (UINT64_MAX - d) / 10) return fail("integer does not fit 64 bits");
            v = v * 10 + d;
            ++p;
        }
        if (p < e && (*p == '.' || *p == 'e' || *p == 'E')) return fail("expected an unsigned integer");
        *out = v;
        return true;
    }
    bool u64_array(std::vector<uint64_t>* out) {
        if (!expect('[')) return false;
        out->clear();
        if (eat(']')) return true;
        do {
            uint64_t v;
            if (!u64(&v)) return false;
            out->push_back(v);
        } while (eat(','));
        return expect(']');
    }
    // any value, ignored (the `__metadata__` object)
    bool skip(int depth = 0) {
        if (depth > 64) return fail("metadata nested too deeply");
        ws();
        if (p >= e) return fail("unexpected end");
        if (*p == '"') {
            std::string s;
            return string(&s);
        }
        if (*p == '{') {
            ++p;
            if (eat('}')) return true;
            do {
                std::string k;
                if (!string(&k) || !expect(':') || !skip(depth + 1)) return false;
            } while (eat(','));
            return expect('}');
        }
        if (*p == '[') {
            ++p;
            if (eat(']')) return true;
            do {
                if (!skip(depth + 1)) return false;
            } while (eat(','));
            return expect(']');
        }
        const uint8_t* s = p;
        while (p < e && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n' && *p != '\r' && *p != '\t') ++p;
        return p > s || fail("expected a value");
    }
};

struct RawTensor {
    uint32_t dtype = 0;
    std::vector<uint64_t> shape;
    uint64_t start = 0, end = 0;
};

bool parse_tensor(Json& j, RawTensor* t) {
    if (!j.expect('{')) return false;
    bool have_dtype = false, have_shape = false, have_off = false;
    if (!j.eat('}')) {
        do {
            std::string key;
            if (!j.string(&key) || !j.expect(':')) return false;
            if (key == "dtype") {
                std::string d;
                if (!j.string(&d)) return false;
                bool found = false;
                for (uint32_t i = 0; i < sizeof(DTYPES) / sizeof(DTYPES[0]); ++i)
                    if (d == DTYPES[i].name) {
                        t->dtype = i;
                        found = true;
                    }
                if (!found) return j.fail("unknown variant `" + d + "`");
                have_dtype = true;
            } else if (key == "shape") {
                if (!j.u64_array(&t->shape)) return false;
                have_shape = true;
            } else if (key == "data_offsets") {
                std::vector<uint64_t> o;
                if (!j.u64_array(&o)) return false;
                if (o.size() != 2) return j.fail("data_offsets must hold two integers");
                t->start = o[0];
                t->end = o[1];
                have_off = true;
            } else if (!j.skip()) {
                return false;
            }
        } while (j.eat(','));
        if (!j.expect('}')) return false;
    }
    if (!have_dtype) return j.fail("missing field `dtype`");
    if (!have_shape) return j.fail("missing field `shape`");
    if (!have_off) return j.fail("missing field `data_offsets`");
    return true;
}

}  // namespace
}  // namespace vyb

using namespace vyb;

struct vyb_safetensors {
    std::string path;
    Digest header_digest{};
    uint64_t file_len = 0, data_start = 0;
    std::vector<Entry> entries;  // canonical (byte-wise) name order
};

extern "C" {

int32_t vyb_safetensors_open(const char* path, vyb_safetensors** out) {
    if (!path || !out) return fail_invalid_program("Fix: pass a shard path and an out-pointer.");
    auto bad = [&](const std::string& what) { return fail_invalid_program("Fix: " + what + "; re-export the checkpoint shard `" + path + "`."); };
    std::unique_ptr<FILE, int (*)(FILE*)> f(std::fopen(path, "rb"), &std::fclose);
    if (!f) return bad(std::string("could not access safetensors shard `") + path + "`");
    if (std::fseek(f.get(), 0, SEEK_END) != 0) return bad("could not access safetensors shard (seek failed)");
    const long long flen = std::ftell(f.get());
    if (flen < 0) return bad("could not access safetensors shard (length unknown)");
    const uint64_t file_len = uint64_t(flen);
    if (file_len < 8) return bad("safetensors shard is " + std::to_string(file_len) + " bytes; expected an 8-byte header prefix");
    std::rewind(f.get());
    uint8_t prefix[8];
    if (std::fread(prefix, 1, 8, f.get()) != 8) return bad("could not read the header prefix");
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | prefix[i];
    if (header_len > MAX_HEADER_BYTES)
        return bad("safetensors header is " + std::to_string(header_len) + " bytes; maximum is " + std::to_string(MAX_HEADER_BYTES));
    const uint64_t data_start = 8 + header_len;
    if (data_start > file_len)
        return bad("safetensors header declares " + std::to_string(header_len) + " bytes but file is " + std::to_string(file_len) + " bytes");
    std::vector<uint8_t> header(header_len);
    if (header_len && std::fread(header.data(), 1, header_len, f.get()) != header_len) return bad("could not read the header");

    Json j{header.data(), header.data() + header.size(), {}, header.data()};
    std::map<std::string, RawTensor> raw;
    bool ok = j.expect('{');
    if (ok && !j.eat('}')) {
        do {
            std::string name;
            if (!(ok = j.string(&name) && j.expect(':'))) break;
            if (name == "__metadata__") {
                if (!(ok = j.skip())) break;
                continue;
            }
            RawTensor t;
            if (!(ok = parse_tensor(j, &t))) break;
            if (!raw.emplace(name, std::move(t)).second) {
                ok = j.fail("duplicate tensor name `" + name + "`");
                break;
            }
        } while (j.eat(','));
        if (ok) ok = j.expect('}');
    }
    if (ok) {
        j.ws();
        if (j.p != j.e) ok = j.fail("trailing characters");
    }
    if (!ok) return bad("invalid safetensors metadata: " + j.err);
    if (raw.size() > MAX_TENSORS)
        return bad("safetensors metadata has " + std::to_string(raw.size()) + " tensors; maximum is " + std::to_string(MAX_TENSORS));

    auto st = std::make_unique<vyb_safetensors>();
    const uint64_t data_len = file_len - data_start;
    std::vector<std::pair<std::pair<uint64_t, uint64_t>, std::string>> ranges;
    for (auto& kv : raw) {
        const std::string& name = kv.first;
        RawTensor& t = kv.second;
        if (name.empty() || name.size() > MAX_TENSOR_NAME_BYTES) return bad("invalid safetensors tensor name `" + name + "`");
        if (t.start > t.end || t.end > data_len)
            return bad("tensor `" + name + "` range [" + std::to_string(t.start) + ", " + std::to_string(t.end) + ") exceeds payload length " +
                       std::to_string(data_len));
        uint64_t elements = 1;
        for (uint64_t extent : t.shape) {
            if (extent && elements > UINT64_MAX / extent) return bad("safetensors tensor shape overflows u64 byte arithmetic");
            elements *= extent;
        }
        const uint64_t width = DTYPES[t.dtype].width;
        if (elements > UINT64_MAX / width) return bad("safetensors tensor shape overflows u64 byte arithmetic");
        if (t.end - t.start != elements * width)
            return bad("tensor `" + name + "` contains " + std::to_string(t.end - t.start) + " bytes; shape and dtype require " +
                       std::to_string(elements * width));
        ranges.push_back({{t.start, t.end}, name});
        Entry e;
        e.name = name;
        e.dtype = t.dtype;
        e.shape = std::move(t.shape);
        e.begin = data_start + t.start;
        e.end = data_start + t.end;
        st->entries.push_back(std::move(e));
    }
    std::sort(ranges.begin(), ranges.end());
    for (size_t i = 1; i < ranges.size(); ++i)
        if (ranges[i - 1].first.second > ranges[i].first.first)
            return bad("safetensors tensor ranges overlap: `" + ranges[i - 1].second + "` and `" + ranges[i].second + "`");
    st->path = path;
    st->file_len = file_len;
    st->data_start = data_start;
    blake3(header.data(), header.size(), st->header_digest.data());
    *out = st.release();
    clear_error();
    return VYB_OK;
}

void vyb_safetensors_free(vyb_safetensors* st) { delete st; }

void vyb_safetensors_identity(const vyb_safetensors* st, uint8_t header_digest[32], uint64_t* file_len, uint64_t* data_start) {
    if (!st) return;
    if (header_digest) std::memcpy(header_digest, st->header_digest.data(), 32);
    if (file_len) *file_len = st->file_len;
    if (data_start) *data_start = st->data_start;
}

uint32_t vyb_safetensors_count(const vyb_safetensors* st) { return st ? uint32_t(st->entries.size()) : 0; }

int32_t vyb_safetensors_entry(const vyb_safetensors* st, uint32_t index, vyb_safetensor_entry* out) {
    if (!st || !out || index >= st->entries.size()) return fail_invalid_program("Fix: tensor index is out of range for this shard.");
    const Entry& e = st->entries[index];
    out->name = e.name.c_str();
    out->dtype = e.dtype;
    out->dtype_name = DTYPES[e.dtype].name;
    out->rank = uint32_t(e.shape.size());
    out->shape = e.shape.data();
    out->file_begin = e.begin;
    out->file_end = e.end;
    return VYB_OK;
}

int32_t vyb_safetensors_find(const vyb_safetensors* st, const char* name, uint32_t* index) {
    if (!st || !name || !index) return fail_invalid_program("Fix: pass a shard, a tensor name and an out-pointer.");
    auto it = std::lower_bound(st->entries.begin(), st->entries.end(), std::string(name),
                               [](const Entry& e, const std::string& n) { return e.name < n; });
    if (it == st->entries.end() || it->name != name)
        return fail_invalid_program(std::string("Fix: the shard holds no tensor named `") + name + "`; check the checkpoint key.");
    *index = uint32_t(it - st->entries.begin());
    return VYB_OK;
}

// SafetensorRequirement (lib.rs:262-271): the compiler's expectation of a tensor, checked before any byte moves
int32_t vyb_safetensors_require(const vyb_safetensors* st, const char* name, const char* dtype_name, const uint64_t* shape, uint32_t rank,
                                uint32_t* index) {
    uint32_t i = 0;
    if (int32_t rc = vyb_safetensors_find(st, name, &i)) return rc;
    const Entry& e = st->entries[i];
    if (!dtype_name || std::string(dtype_name) != DTYPES[e.dtype].name)
        return fail_invalid_program(std::string("Fix: tensor `") + name + "` is stored as " + DTYPES[e.dtype].name + ", the model requires " +
                                    (dtype_name ? dtype_name : "(null)") + "; convert the checkpoint or fix the requirement.");
    if (e.shape.size() != rank || (rank && !shape) || !std::equal(e.shape.begin(), e.shape.end(), shape))
        return fail_invalid_program(std::string("Fix: tensor `") + name + "` has a different shape than the model requires; check the checkpoint key.");
    if (index) *index = i;
    return VYB_OK;
}

// The tensor's bytes, file -> resident device buffer at `dst_offset`, in bounded pieces (no whole-tensor host copy).
int32_t vyb_safetensors_upload(const vyb_safetensors* st, uint32_t index, vyb_device* device, vyb_resident_handle handle, uint64_t dst_offset) {
    if (!st || !device || index >= st->entries.size()) return fail_invalid_program("Fix: pass a shard, a device and a tensor index inside the shard.");
    const Entry& e = st->entries[index];
    std::unique_ptr<FILE, int (*)(FILE*)> f(std::fopen(st->path.c_str(), "rb"), &std::fclose);
    if (!f) return fail_invalid_program("Fix: could not access safetensors shard `" + st->path + "` again; it was moved or removed after it was indexed.");
    std::fseek(f.get(), 0, SEEK_END);
    if (uint64_t(std::ftell(f.get())) != st->file_len)
        return fail_invalid_program("Fix: safetensors shard `" + st->path + "` changed length after it was indexed; index it again.");
    if (std::fseek(f.get(), long(e.begin), SEEK_SET) != 0) return fail_invalid_program("Fix: could not seek inside the safetensors shard.");
    std::vector<uint8_t> piece(std::min<uint64_t>(e.end - e.begin, 16ull << 20));
    for (uint64_t done = 0, total = e.end - e.begin; done < total;) {
        const size_t n = size_t(std::min<uint64_t>(piece.size(), total - done));
        if (std::fread(piece.data(), 1, n, f.get()) != n)
            return fail_invalid_program("Fix: safetensors shard `" + st->path + "` ended inside tensor `" + e.name + "`; index it again.");
        if (int32_t rc = vyb_upload_at(device, handle, dst_offset + done, piece.data(), n)) return rc;
        done += n;
    }
    return VYB_OK;
}

}  // extern "C"
