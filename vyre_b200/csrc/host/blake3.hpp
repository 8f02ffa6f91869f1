#pragma once
#include <cstddef>
#include <cstdint>

namespace vyb {
// 32-byte BLAKE3 hash (unkeyed) of `len` bytes.
void blake3(const void* data, size_t len, uint8_t out[32]);
}  // namespace vyb
