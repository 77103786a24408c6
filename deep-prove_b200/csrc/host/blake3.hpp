// BLAKE3 (hash mode, 32-byte digest) for the host-side Fiat-Shamir transcript.
// Written from the published specification; portable C++, no SIMD: transcript
// inputs are a few hundred bytes per sumcheck round.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

namespace dpb {
namespace blake3 {

constexpr uint32_t kIV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                             0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
constexpr uint8_t kSchedule[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum : uint32_t { kChunkStart = 1, kChunkEnd = 2, kParent = 4, kRoot = 8 };
constexpr size_t kBlock = 64, kChunk = 1024;

inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

inline void mix(uint32_t* v, int a, int b, int c, int d, uint32_t x, uint32_t y) {
    v[a] += v[b] + x;
    v[d] = rotr(v[d] ^ v[a], 16);
    v[c] += v[d];
    v[b] = rotr(v[b] ^ v[c], 12);
    v[a] += v[b] + y;
    v[d] = rotr(v[d] ^ v[a], 8);
    v[c] += v[d];
    v[b] = rotr(v[b] ^ v[c], 7);
}

// One compression; writes the 8-word chaining value to out.
inline void compress(const uint32_t cv[8], const uint8_t block[kBlock], uint64_t counter,
                     uint32_t block_len, uint32_t flags, uint32_t out[8]) {
    uint32_t m[16], v[16];
    for (int i = 0; i < 16; i++)
        m[i] = (uint32_t)block[4 * i] | ((uint32_t)block[4 * i + 1] << 8) |
               ((uint32_t)block[4 * i + 2] << 16) | ((uint32_t)block[4 * i + 3] << 24);
    for (int i = 0; i < 8; i++) v[i] = cv[i];
    for (int i = 0; i < 4; i++) v[8 + i] = kIV[i];
    v[12] = (uint32_t)counter;
    v[13] = (uint32_t)(counter >> 32);
    v[14] = block_len;
    v[15] = flags;
    for (int r = 0; r < 7; r++) {
        mix(v, 0, 4, 8, 12, m[0], m[1]);
        mix(v, 1, 5, 9, 13, m[2], m[3]);
        mix(v, 2, 6, 10, 14, m[4], m[5]);
        mix(v, 3, 7, 11, 15, m[6], m[7]);
        mix(v, 0, 5, 10, 15, m[8], m[9]);
        mix(v, 1, 6, 11, 12, m[10], m[11]);
        mix(v, 2, 7, 8, 13, m[12], m[13]);
        mix(v, 3, 4, 9, 14, m[14], m[15]);
        if (r < 6) {
            uint32_t t[16];
            for (int i = 0; i < 16; i++) t[i] = m[kSchedule[i]];
            memcpy(m, t, sizeof m);
        }
    }
    for (int i = 0; i < 8; i++) out[i] = v[i] ^ v[i + 8];
}

// Chaining value of one chunk (<= 1024 bytes).
inline void chunk_cv(const uint8_t* data, size_t len, uint64_t index, bool root, uint32_t out[8]) {
    uint32_t cv[8];
    memcpy(cv, kIV, sizeof cv);
    const size_t n_blocks = len == 0 ? 1 : (len + kBlock - 1) / kBlock;
    for (size_t b = 0; b < n_blocks; b++) {
        uint8_t block[kBlock] = {0};
        const size_t off = b * kBlock;
        const size_t bl = len - off < kBlock ? len - off : kBlock;
        if (bl) memcpy(block, data + off, bl);
        uint32_t flags = 0;
        if (b == 0) flags |= kChunkStart;
        if (b + 1 == n_blocks) flags |= kChunkEnd | (root ? kRoot : 0u);
        uint32_t next[8];
        compress(cv, block, index, (uint32_t)bl, flags, next);
        memcpy(cv, next, sizeof cv);
    }
    memcpy(out, cv, sizeof cv);
}

// Chaining value of a subtree; the left child takes the largest power-of-two
// number of chunks that leaves at least one byte for the right child.
inline void subtree_cv(const uint8_t* data, size_t len, uint64_t first_chunk, bool root, uint32_t out[8]) {
    if (len <= kChunk) {
        chunk_cv(data, len, first_chunk, root, out);
        return;
    }
    const size_t n_chunks = (len + kChunk - 1) / kChunk;
    size_t left = 1;
    while (left * 2 < n_chunks) left *= 2;
    uint32_t l[8], r[8];
    subtree_cv(data, left * kChunk, first_chunk, false, l);
    subtree_cv(data + left * kChunk, len - left * kChunk, first_chunk + left, false, r);
    uint8_t block[kBlock];
    for (int i = 0; i < 8; i++) {
        for (int b = 0; b < 4; b++) {
            block[4 * i + b] = (uint8_t)(l[i] >> (8 * b));
            block[32 + 4 * i + b] = (uint8_t)(r[i] >> (8 * b));
        }
    }
    compress(kIV, block, 0, kBlock, kParent | (root ? kRoot : 0u), out);
}

inline void hash(const uint8_t* data, size_t len, uint8_t out[32]) {
    uint32_t cv[8];
    subtree_cv(data, len, 0, true, cv);
    for (int i = 0; i < 8; i++)
        for (int b = 0; b < 4; b++) out[4 * i + b] = (uint8_t)(cv[i] >> (8 * b));
}

}  // namespace blake3
}  // namespace dpb
