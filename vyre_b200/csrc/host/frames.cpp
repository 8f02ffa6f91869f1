// The reference's authenticated wire frames around this backend's target bytes.
//
// vyre-megakernel frames all three layers the same way (lib.rs:1326-1355 for the neutral artifact, envelope.rs:763-860
// for target payloads and envelopes):
//
//     magic[4] | schema_version u16 LE | body_len u32 LE | body (compact serde_json) | BLAKE3(domain | schema_version
//     u16 LE | body_len u64 LE | body)[32]
//
//     VMK0  schema 4  domain "vyre-megakernel-artifact-v4\0"        neutral artifact (lib.rs:52-59)
//     VTP0  schema 3  domain "vyre-megakernel-target-payload-v3\0"  target payload   (envelope.rs:10-19)
//     VME0  schema 2  domain "vyre-megakernel-envelope-v2\0"        envelope         (envelope.rs:10-19)
//
// Built here: the framing itself for all three (encode, and decode with the reference's checks in its order: length,
// magic, schema, declared length, digest); the VTP0 body of THIS backend's payload (TargetPayloadBody, envelope.rs:182-192:
// schema_version, neutral_artifact as 32 numbers, format, profile, entries sorted by name with bindings sorted by
// (group, slot), bytes as numbers; the opaque `bytes` are the payload's own sealed bytes) and its way back; the VME0 body
// (EnvelopeBody, envelope.rs:383-389: the neutral artifact's frame and the payload frames as byte arrays) with the check
// that every payload names the digest of the neutral frame it travels with. The VMK0 BODY is the reference compiler's
// own output (nodes, plan, ABI, resources, provenance); it is authenticated and carried, not produced or interpreted.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "blake3.hpp"
#include "model.hpp"

using namespace vyb;

namespace {

struct Layer {
    const char* magic;
    uint16_t schema;
    const char* domain;  // the trailing NUL is part of the domain
    size_t domain_len;
    const char* path;
};
const Layer LAYERS[3] = {
    {"VMK0", 4, "vyre-megakernel-artifact-v4", 28, "artifact"},
    {"VTP0", 3, "vyre-megakernel-target-payload-v3", 34, "target_payload"},
    {"VME0", 2, "vyre-megakernel-envelope-v2", 28, "envelope"},
};
constexpr size_t HEADER = 10, DIGEST = 32;

void frame_digest(const Layer& l, const uint8_t* body, size_t len, uint8_t out[32]) {
    std::vector<uint8_t> buf;
    buf.reserve(l.domain_len + 10 + len);
    buf.insert(buf.end(), l.domain, l.domain + l.domain_len);  // includes the NUL that ends the literal
    buf.push_back(uint8_t(l.schema & 0xFF));
    buf.push_back(uint8_t(l.schema >> 8));
    for (int i = 0; i < 8; ++i) buf.push_back(uint8_t((uint64_t(len) >> (8 * i)) & 0xFF));
    buf.insert(buf.end(), body, body + len);
    vyb_blake3(buf.data(), buf.size(), out);
}

int32_t malformed(const Layer& l, const char* field, const std::string& what, const char* fix) {
    return fail_invalid_program(std::string(l.path) + "." + field + ": " + what + ". Fix: " + fix);
}

std::vector<uint8_t> encode(const Layer& l, const uint8_t* body, size_t len) {
    std::vector<uint8_t> f;
    f.reserve(HEADER + len + DIGEST);
    f.insert(f.end(), l.magic, l.magic + 4);
    f.push_back(uint8_t(l.schema & 0xFF));
    f.push_back(uint8_t(l.schema >> 8));
    for (int i = 0; i < 4; ++i) f.push_back(uint8_t((uint32_t(len) >> (8 * i)) & 0xFF));
    f.insert(f.end(), body, body + len);
    uint8_t d[32];
    frame_digest(l, body, len, d);
    f.insert(f.end(), d, d + 32);
    return f;
}

// envelope.rs:788-860, in its order
int32_t decode(const Layer& l, const uint8_t* f, size_t n, const uint8_t** body, size_t* body_len, uint8_t digest[32]) {
    if (n < HEADER + DIGEST)
        return malformed(l, "header", "framed bytes are shorter than the fixed header and digest", "supply one complete canonical frame");
    if (std::memcmp(f, l.magic, 4) != 0)
        return malformed(l, "magic", "framing magic is invalid", "supply bytes emitted for the expected artifact layer");
    const uint16_t version = uint16_t(f[4] | (f[5] << 8));
    if (version != l.schema)
        return malformed(l, "schema_version", "schema " + std::to_string(version) + " is unsupported; expected " + std::to_string(l.schema),
                         "recompile or re-materialize with a compatible schema version");
    const size_t len = size_t(f[6]) | (size_t(f[7]) << 8) | (size_t(f[8]) << 16) | (size_t(f[9]) << 24);
    const size_t expected = HEADER + len + DIGEST;
    if (n != expected)
        return malformed(l, "body_length", "framing declares " + std::to_string(expected) + " bytes but received " + std::to_string(n),
                         "supply exactly one complete canonical frame");
    uint8_t d[32];
    frame_digest(l, f + HEADER, len, d);
    if (std::memcmp(d, f + HEADER + len, 32) != 0)
        return malformed(l, "digest", "framed body does not match its content identity", "discard the corrupted bytes and regenerate them");
    if (body) *body = f + HEADER;
    if (body_len) *body_len = len;
    if (digest) std::memcpy(digest, d, 32);
    return VYB_OK;
}

int32_t hand_out(const std::vector<uint8_t>& v, uint8_t** frame, size_t* len) {
    uint8_t* p = static_cast<uint8_t*>(std::malloc(v.size() ? v.size() : 1));
    if (!p) return fail_oom(v.size(), 0);
    std::memcpy(p, v.data(), v.size());
    *frame = p;
    *len = v.size();
    clear_error();
    return VYB_OK;
}

// ---- compact JSON, serde_json's form: no spaces, fields in declaration order ---------------------------------------------
void put_bytes(std::string& s, const uint8_t* b, size_t n) {
    s.push_back('[');
    for (size_t i = 0; i < n; ++i) {
        if (i) s.push_back(',');
        s += std::to_string(unsigned(b[i]));
    }
    s.push_back(']');
}
void put_string(std::string& s, const std::string& v) {
    s.push_back('"');
    for (unsigned char c : v) {
        if (c == '"' || c == '\\') {
            s.push_back('\\');
            s.push_back(char(c));
        } else if (c < 0x20) {
            char buf[8];
            std::snprintf(buf, sizeof buf, "\\u%04x", c);
            s += buf;
        } else {
            s.push_back(char(c));
        }
    }
    s.push_back('"');
}
void put_u3(std::string& s, const uint32_t* v) {
    s += "[" + std::to_string(v[0]) + "," + std::to_string(v[1]) + "," + std::to_string(v[2]) + "]";
}

// a reader for the same subset: objects, arrays, strings with the escapes above, unsigned integers
struct Reader {
    const uint8_t* p;
    const uint8_t* e;
    bool ok = true;
    bool eat(char c) {
        if (p < e && *p == uint8_t(c)) {
            ++p;
            return true;
        }
        return false;
    }
    void need(char c) {
        if (!eat(c)) ok = false;
    }
    std::string key() {
        std::string k = string();
        need(':');
        return k;
    }
    std::string string() {
        std::string out;
        if (!eat('"')) {
            ok = false;
            return out;
        }
        while (p < e && *p != '"') {
            if (*p == '\\' && p + 1 < e) {
                ++p;
                if (*p == 'u' && p + 4 < e) {
                    out.push_back(char(std::strtoul(std::string(reinterpret_cast<const char*>(p + 1), 4).c_str(), nullptr, 16)));
                    p += 4;
                } else {
                    out.push_back(char(*p));
                }
                ++p;
            } else {
                out.push_back(char(*p++));
            }
        }
        need('"');
        return out;
    }
    uint64_t number() {
        if (p >= e || *p < '0' || *p > '9') {
            ok = false;
            return 0;
        }
        uint64_t v = 0;
        while (p < e && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
        return v;
    }
    std::vector<uint8_t> bytes() {
        std::vector<uint8_t> out;
        need('[');
        if (eat(']')) return out;
        do {
            const uint64_t v = number();
            if (v > 255) ok = false;
            out.push_back(uint8_t(v));
        } while (ok && eat(','));
        need(']');
        return out;
    }
    void u3(uint32_t* v) {
        need('[');
        for (int i = 0; i < 3; ++i) {
            if (i) need(',');
            v[i] = uint32_t(number());
        }
        need(']');
    }
    void expect_key(const char* name) {
        if (key() != name) ok = false;
    }
};

const char* access_name(uint32_t access) {
    return access == VYB_ACCESS_READ_ONLY ? "read_only" : access == VYB_ACCESS_OUTPUT ? "write_only" : "read_write";
}

}  // namespace

extern "C" {

int32_t vyb_frame_encode(uint32_t layer, const uint8_t* body, size_t body_len, uint8_t** frame, size_t* frame_len) {
    if (layer > 2 || (!body && body_len) || !frame || !frame_len)
        return fail_invalid_program("Fix: pass a layer (0 VMK0, 1 VTP0, 2 VME0), a body and output pointers.");
    if (body_len > 0xFFFFFFFFull)
        return fail_invalid_program("envelope.body: canonical body exceeds the u32 framing limit. Fix: reduce or detach target payload bytes");
    return hand_out(encode(LAYERS[layer], body, body_len), frame, frame_len);
}

int32_t vyb_frame_decode(uint32_t layer, const uint8_t* frame, size_t frame_len, const uint8_t** body, size_t* body_len,
                         uint8_t digest[32]) {
    if (layer > 2 || !frame) return fail_invalid_program("Fix: pass a layer (0 VMK0, 1 VTP0, 2 VME0) and the framed bytes.");
    const int32_t rc = decode(LAYERS[layer], frame, frame_len, body, body_len, digest);
    if (rc == VYB_OK) clear_error();
    return rc;
}

void vyb_frame_free(uint8_t* frame) { std::free(frame); }

int32_t vyb_payload_to_vtp0(const vyb_payload* payload, const uint8_t neutral_artifact[32], uint32_t node_id,
                            const uint32_t* value_ids, uint32_t n_value_ids, uint8_t** frame, size_t* frame_len) {
    if (!payload || !neutral_artifact || !frame || !frame_len)
        return fail_invalid_program("Fix: pass a payload, the neutral artifact's digest and output pointers.");
    const Payload& p = payload->p;
    if (p.bytes.empty())
        return fail_invalid_program("target_payload.bytes: target payload bytes are empty. Fix: attach non-empty bytes emitted for the declared target format");
    std::string s = "{\"schema_version\":3,\"neutral_artifact\":";
    put_bytes(s, neutral_artifact, 32);
    s += ",\"format\":{\"identity\":";
    put_string(s, p.format);
    s += ",\"version\":" + std::to_string(p.format_version) + "},\"profile\":{\"identity\":";
    put_string(s, std::string(p.profile.identity, strnlen(p.profile.identity, sizeof p.profile.identity)));
    s += ",\"generation\":" + std::to_string(p.profile.generation) + ",\"max_workgroup_size\":";
    put_u3(s, p.profile.max_workgroup_size);
    s += ",\"max_invocations_per_workgroup\":" + std::to_string(p.profile.max_invocations) +
         ",\"max_dynamic_shared_bytes\":" + std::to_string(p.profile.max_dynamic_shared_bytes) +
         ",\"subgroup_size\":" + std::to_string(p.profile.subgroup_size) + "},\"entries\":[";
    std::vector<const TargetModule*> mods;
    for (const TargetModule& m : p.modules) mods.push_back(&m);
    std::sort(mods.begin(), mods.end(), [](const TargetModule* a, const TargetModule* b) { return a->entry_point < b->entry_point; });
    for (size_t mi = 0; mi < mods.size(); ++mi) {
        const TargetModule& m = *mods[mi];
        Program prog;
        std::string err;
        if (!Program::from_wire(m.program_wire.data(), m.program_wire.size(), &prog, &err))
            return fail_invalid_program("Fix: the payload's module does not hold a readable program: " + err);
        std::vector<const BufferDecl*> decls;
        for (const BufferDecl& b : prog.buffers)
            if (b.access != VYB_ACCESS_WORKGROUP) decls.push_back(&b);
        if (value_ids && n_value_ids != decls.size())
            return fail_invalid_program("Fix: pass one ArtifactValueId per bound buffer (" + std::to_string(decls.size()) + "), got " +
                                        std::to_string(n_value_ids) + ".");
        std::vector<size_t> order(decls.size());
        for (size_t i = 0; i < order.size(); ++i) order[i] = i;
        std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return decls[a]->binding < decls[b]->binding; });
        if (mi) s.push_back(',');
        s += "{\"name\":";
        put_string(s, m.entry_point);
        s += ",\"node\":" + std::to_string(node_id) + ",\"workgroup_size\":";
        put_u3(s, m.workgroup.data());
        s += ",\"grid_size\":";
        put_u3(s, m.grid.data());
        s += ",\"dynamic_shared_bytes\":" + std::to_string(m.dynamic_shared_bytes) + ",\"resource_bindings\":[";
        for (size_t oi = 0; oi < order.size(); ++oi) {
            const BufferDecl& b = *decls[order[oi]];
            if (oi) s.push_back(',');
            s += "{\"resource\":" + std::to_string(value_ids ? value_ids[order[oi]] : b.binding) + ",\"group\":0,\"slot\":" +
                 std::to_string(b.binding) + ",\"memory\":\"global\",\"access\":\"" + access_name(b.access) + "\"}";
        }
        s += "]}";
    }
    s += "],\"bytes\":";
    put_bytes(s, p.bytes.data(), p.bytes.size());
    s.push_back('}');
    if (s.size() > 0xFFFFFFFFull)
        return fail_invalid_program("envelope.body: canonical body exceeds the u32 framing limit. Fix: reduce or detach target payload bytes");
    return hand_out(encode(LAYERS[1], reinterpret_cast<const uint8_t*>(s.data()), s.size()), frame, frame_len);
}

int32_t vyb_payload_from_vtp0(const uint8_t* frame, size_t frame_len, vyb_payload** payload, uint8_t neutral_artifact[32]) {
    if (!frame || !payload) return fail_invalid_program("Fix: pass the framed bytes and an output pointer.");
    const uint8_t* body = nullptr;
    size_t len = 0;
    if (int32_t rc = decode(LAYERS[1], frame, frame_len, &body, &len, nullptr)) return rc;
    auto bad = [&](const char* what) {
        return fail_invalid_program(std::string("target_payload.body: ") + what +
                                    ". Fix: supply canonical target payload bytes emitted by this crate");
    };
    Reader r{body, body + len};
    r.need('{');
    r.expect_key("schema_version");
    const uint64_t schema = r.number();
    r.need(',');
    r.expect_key("neutral_artifact");
    const std::vector<uint8_t> neutral = r.bytes();
    r.need(',');
    r.expect_key("format");
    r.need('{');
    r.expect_key("identity");
    const std::string identity = r.string();
    r.need(',');
    r.expect_key("version");
    const uint64_t version = r.number();
    r.need('}');
    if (!r.ok) return bad("the head of the body is not a TargetPayloadBody");
    if (schema != 3) return bad("body schema differs from the frame's");
    if (neutral.size() != 32) return bad("neutral_artifact is not a 32-byte digest");
    // profile and entries are re-derived from the target bytes themselves; find `bytes`, the last field
    static const char KEY[] = ",\"bytes\":[";
    const uint8_t* at = nullptr;
    for (const uint8_t* q = body + len - 1; q >= r.p + sizeof KEY - 1; --q)
        if (*q == '[' && std::memcmp(q - (sizeof KEY - 2), KEY, sizeof KEY - 1) == 0) {
            at = q;
            break;
        }
    if (!at) return bad("no `bytes` field");
    Reader br{at, body + len};
    const std::vector<uint8_t> bytes = br.bytes();
    br.need('}');
    if (!br.ok || br.p != body + len) return bad("`bytes` is not the closing byte array");
    if (bytes.empty()) return bad("target payload bytes are empty");
    vyb_payload* out = nullptr;
    if (int32_t rc = vyb_payload_from_bytes(bytes.data(), bytes.size(), &out)) return rc;
    if (out->p.format != identity || out->p.format_version != version) {
        vyb_payload_free(out);
        return bad("format identity or version differs from the one sealed in the target bytes");
    }
    if (neutral_artifact) std::memcpy(neutral_artifact, neutral.data(), 32);
    *payload = out;
    clear_error();
    return VYB_OK;
}

int32_t vyb_envelope_to_vme0(const uint8_t* vmk0, size_t vmk0_len, const uint8_t* const* vtp0, const size_t* vtp0_len,
                             uint32_t n_payloads, uint8_t** frame, size_t* frame_len) {
    if (!vmk0 || (n_payloads && (!vtp0 || !vtp0_len)) || !frame || !frame_len)
        return fail_invalid_program("Fix: pass the neutral artifact's frame, the payload frames and output pointers.");
    uint8_t neutral[32];
    if (int32_t rc = decode(LAYERS[0], vmk0, vmk0_len, nullptr, nullptr, neutral)) return rc;
    std::string s = "{\"schema_version\":2,\"neutral_artifact\":";
    put_bytes(s, vmk0, vmk0_len);
    s += ",\"target_payloads\":[";
    for (uint32_t i = 0; i < n_payloads; ++i) {
        const uint8_t* body = nullptr;
        size_t len = 0;
        if (int32_t rc = decode(LAYERS[1], vtp0[i], vtp0_len[i], &body, &len, nullptr)) return rc;
        Reader r{body, body + len};
        r.need('{');
        r.expect_key("schema_version");
        r.number();
        r.need(',');
        r.expect_key("neutral_artifact");
        const std::vector<uint8_t> named = r.bytes();
        if (!r.ok || named.size() != 32 || std::memcmp(named.data(), neutral, 32) != 0)
            return fail_invalid_program("envelope.target_payloads[" + std::to_string(i) +
                                        "]: target payload is bound to another neutral artifact. Fix: attach payloads compiled for this artifact");
        if (i) s.push_back(',');
        put_bytes(s, vtp0[i], vtp0_len[i]);
    }
    s += "]}";
    if (s.size() > 0xFFFFFFFFull)
        return fail_invalid_program("envelope.body: canonical body exceeds the u32 framing limit. Fix: reduce or detach target payload bytes");
    return hand_out(encode(LAYERS[2], reinterpret_cast<const uint8_t*>(s.data()), s.size()), frame, frame_len);
}

int32_t vyb_envelope_from_vme0(const uint8_t* frame, size_t frame_len, uint32_t index, uint8_t** inner, size_t* inner_len,
                               uint32_t* n_payloads) {
    if (!frame) return fail_invalid_program("Fix: pass the framed bytes.");
    const uint8_t* body = nullptr;
    size_t len = 0;
    if (int32_t rc = decode(LAYERS[2], frame, frame_len, &body, &len, nullptr)) return rc;
    auto bad = [&](const char* what) {
        return fail_invalid_program(std::string("envelope.body: ") + what + ". Fix: supply canonical envelope bytes emitted by this crate");
    };
    Reader r{body, body + len};
    r.need('{');
    r.expect_key("schema_version");
    if (r.number() != 2) return bad("body schema differs from the frame's");
    r.need(',');
    r.expect_key("neutral_artifact");
    std::vector<std::vector<uint8_t>> parts;
    parts.push_back(r.bytes());
    r.need(',');
    r.expect_key("target_payloads");
    r.need('[');
    if (!r.eat(']')) {
        do parts.push_back(r.bytes());
        while (r.ok && r.eat(','));
        r.need(']');
    }
    r.need('}');
    if (!r.ok || r.p != body + len) return bad("not an EnvelopeBody");
    uint8_t neutral[32];
    if (int32_t rc = decode(LAYERS[0], parts[0].data(), parts[0].size(), nullptr, nullptr, neutral)) return rc;
    for (size_t i = 1; i < parts.size(); ++i)
        if (int32_t rc = decode(LAYERS[1], parts[i].data(), parts[i].size(), nullptr, nullptr, nullptr)) return rc;
    if (n_payloads) *n_payloads = uint32_t(parts.size() - 1);
    if (inner && inner_len) {
        if (index >= parts.size()) return fail_invalid_program("Fix: index 0 is the neutral artifact, 1.." + std::to_string(parts.size() - 1) + " the payloads.");
        return hand_out(parts[index], inner, inner_len);
    }
    clear_error();
    return VYB_OK;
}

}  // extern "C"
