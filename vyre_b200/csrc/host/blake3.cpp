// BLAKE3 (unkeyed hash mode, 32-byte output) written from the published specification.
// vyre authenticates Artifact and TargetPayload identities with blake3
// (vyre-megakernel/src/lib.rs:52-59, envelope.rs:14-19); the native backend must produce the same digests
// from the same bytes, so it carries its own implementation instead of a different hash.
#include "blake3.hpp"

#include <cstring>

namespace vyb {
namespace {

constexpr uint32_t IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                            0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
constexpr uint8_t MSG_PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
constexpr uint32_t CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8;
constexpr size_t BLOCK_LEN = 64, CHUNK_LEN = 1024;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

inline void g(uint32_t* s, int a, int b, int c, int d, uint32_t mx, uint32_t my) {
    s[a] = s[a] + s[b] + mx;
    s[d] = rotr(s[d] ^ s[a], 16);
    s[c] = s[c] + s[d];
    s[b] = rotr(s[b] ^ s[c], 12);
    s[a] = s[a] + s[b] + my;
    s[d] = rotr(s[d] ^ s[a], 8);
    s[c] = s[c] + s[d];
    s[b] = rotr(s[b] ^ s[c], 7);
}

inline void round_fn(uint32_t* s, const uint32_t* m) {
    g(s, 0, 4, 8, 12, m[0], m[1]);
    g(s, 1, 5, 9, 13, m[2], m[3]);
    g(s, 2, 6, 10, 14, m[4], m[5]);
    g(s, 3, 7, 11, 15, m[6], m[7]);
    g(s, 0, 5, 10, 15, m[8], m[9]);
    g(s, 1, 6, 11, 12, m[10], m[11]);
    g(s, 2, 7, 8, 13, m[12], m[13]);
    g(s, 3, 4, 9, 14, m[14], m[15]);
}

// Full 16-word compression output (the first 8 words are the chaining value).
void compress(const uint32_t cv[8], const uint32_t block_words[16], uint64_t counter, uint32_t block_len,
              uint32_t flags, uint32_t out[16]) {
    uint32_t s[16] = {cv[0], cv[1], cv[2], cv[3], cv[4], cv[5], cv[6], cv[7],
                      IV[0], IV[1], IV[2], IV[3], uint32_t(counter), uint32_t(counter >> 32), block_len, flags};
    uint32_t m[16];
    std::memcpy(m, block_words, sizeof(m));
    for (int r = 0; r < 7; ++r) {
        round_fn(s, m);
        if (r < 6) {
            uint32_t p[16];
            for (int i = 0; i < 16; ++i) p[i] = m[MSG_PERM[i]];
            std::memcpy(m, p, sizeof(m));
        }
    }
    for (int i = 0; i < 8; ++i) {
        s[i] ^= s[i + 8];
        s[i + 8] ^= cv[i];
    }
    std::memcpy(out, s, sizeof(s));
}

inline void words_from_le(const uint8_t* bytes, size_t len, uint32_t words[16]) {
    uint8_t block[BLOCK_LEN] = {0};
    std::memcpy(block, bytes, len);
    for (int i = 0; i < 16; ++i)
        words[i] = uint32_t(block[4 * i]) | (uint32_t(block[4 * i + 1]) << 8) | (uint32_t(block[4 * i + 2]) << 16) |
                   (uint32_t(block[4 * i + 3]) << 24);
}

// Pending final compression of a subtree: kept un-applied so ROOT can be added if it is the last one.
struct Output {
    uint32_t cv[8];
    uint32_t block[16];
    uint64_t counter;
    uint32_t block_len;
    uint32_t flags;
    void chaining_value(uint32_t out[8]) const {
        uint32_t full[16];
        compress(cv, block, counter, block_len, flags, full);
        std::memcpy(out, full, 32);
    }
    void root_bytes(uint8_t out[32]) const {
        uint32_t full[16];
        compress(cv, block, 0, block_len, flags | ROOT, full);
        for (int i = 0; i < 8; ++i) {
            out[4 * i] = uint8_t(full[i]);
            out[4 * i + 1] = uint8_t(full[i] >> 8);
            out[4 * i + 2] = uint8_t(full[i] >> 16);
            out[4 * i + 3] = uint8_t(full[i] >> 24);
        }
    }
};

Output chunk_output(const uint8_t* data, size_t len, uint64_t chunk_counter) {
    uint32_t cv[8];
    std::memcpy(cv, IV, sizeof(cv));
    size_t blocks = len == 0 ? 1 : (len + BLOCK_LEN - 1) / BLOCK_LEN;
    Output o{};
    for (size_t b = 0; b < blocks; ++b) {
        size_t off = b * BLOCK_LEN;
        size_t bl = len - off < BLOCK_LEN ? len - off : BLOCK_LEN;
        uint32_t words[16];
        words_from_le(data + off, bl, words);
        uint32_t flags = (b == 0 ? CHUNK_START : 0) | (b + 1 == blocks ? CHUNK_END : 0);
        if (b + 1 == blocks) {
            std::memcpy(o.cv, cv, sizeof(cv));
            std::memcpy(o.block, words, sizeof(words));
            o.counter = chunk_counter;
            o.block_len = uint32_t(bl);
            o.flags = flags;
        } else {
            uint32_t full[16];
            compress(cv, words, chunk_counter, uint32_t(bl), flags, full);
            std::memcpy(cv, full, 32);
        }
    }
    return o;
}

Output parent_output(const uint32_t left[8], const uint32_t right[8]) {
    Output o{};
    std::memcpy(o.cv, IV, sizeof(IV));
    std::memcpy(o.block, left, 32);
    std::memcpy(o.block + 8, right, 32);
    o.counter = 0;
    o.block_len = BLOCK_LEN;
    o.flags = PARENT;
    return o;
}

}  // namespace

void blake3(const void* data_v, size_t len, uint8_t out[32]) {
    const uint8_t* data = static_cast<const uint8_t*>(data_v);
    // Incremental left-to-right hashing with a stack of completed subtree chaining values: after chunk
    // number t (1-based) is finished, merge once per trailing zero bit of t.
    uint32_t stack[54][8];
    int depth = 0;
    size_t total_chunks = len == 0 ? 1 : (len + CHUNK_LEN - 1) / CHUNK_LEN;
    Output last{};
    for (size_t c = 0; c < total_chunks; ++c) {
        size_t off = c * CHUNK_LEN;
        size_t cl = len - off < CHUNK_LEN ? len - off : CHUNK_LEN;
        Output co = chunk_output(data + off, cl, c);
        if (c + 1 == total_chunks) {
            last = co;
            break;
        }
        uint32_t cv[8];
        co.chaining_value(cv);
        uint64_t done = c + 1;
        while ((done & 1) == 0) {
            Output p = parent_output(stack[depth - 1], cv);
            p.chaining_value(cv);
            --depth;
            done >>= 1;
        }
        std::memcpy(stack[depth++], cv, 32);
    }
    // Fold the remaining stack from the top: each level is parent(stack entry, current).
    Output cur = last;
    while (depth > 0) {
        uint32_t cv[8];
        cur.chaining_value(cv);
        cur = parent_output(stack[depth - 1], cv);
        --depth;
    }
    cur.root_bytes(out);
}

}  // namespace vyb
