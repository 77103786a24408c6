"""BLAKE3 (hash mode, 32-byte output) in pure Python, from the published
specification.  TEST INFRASTRUCTURE ONLY: the oracle's transcript uses it so
that the checker shares no code with the library's own C++ BLAKE3.  Inputs are
a few hundred bytes per call, so speed is irrelevant.
"""
import struct

IV = (0x6A09E667, 0xBB67AE85, 0x3C6EF372, 0xA54FF53A, 0x510E527F, 0x9B05688C, 0x1F83D9AB, 0x5BE0CD19)
PERM = (2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8)
CHUNK_START, CHUNK_END, PARENT, ROOT = 1, 2, 4, 8
M32 = 0xFFFFFFFF


def _rotr(x, n):
    return ((x >> n) | (x << (32 - n))) & M32


def _g(s, a, b, c, d, mx, my):
    s[a] = (s[a] + s[b] + mx) & M32
    s[d] = _rotr(s[d] ^ s[a], 16)
    s[c] = (s[c] + s[d]) & M32
    s[b] = _rotr(s[b] ^ s[c], 12)
    s[a] = (s[a] + s[b] + my) & M32
    s[d] = _rotr(s[d] ^ s[a], 8)
    s[c] = (s[c] + s[d]) & M32
    s[b] = _rotr(s[b] ^ s[c], 7)


def _compress(cv, block_words, counter, block_len, flags):
    s = list(cv) + list(IV[:4]) + [counter & M32, (counter >> 32) & M32, block_len, flags]
    m = list(block_words)
    for rnd in range(7):
        _g(s, 0, 4, 8, 12, m[0], m[1])
        _g(s, 1, 5, 9, 13, m[2], m[3])
        _g(s, 2, 6, 10, 14, m[4], m[5])
        _g(s, 3, 7, 11, 15, m[6], m[7])
        _g(s, 0, 5, 10, 15, m[8], m[9])
        _g(s, 1, 6, 11, 12, m[10], m[11])
        _g(s, 2, 7, 8, 13, m[12], m[13])
        _g(s, 3, 4, 9, 14, m[14], m[15])
        if rnd < 6:
            m = [m[PERM[i]] for i in range(16)]
    return [s[i] ^ s[i + 8] for i in range(8)]


def _words(block):
    return struct.unpack("<16I", block.ljust(64, b"\0"))


def _chunk_cv(chunk, index, root):
    cv = IV
    blocks = [chunk[i:i + 64] for i in range(0, len(chunk), 64)] or [b""]
    for i, blk in enumerate(blocks):
        flags = 0
        if i == 0:
            flags |= CHUNK_START
        if i == len(blocks) - 1:
            flags |= CHUNK_END
            if root:
                flags |= ROOT
        cv = _compress(cv, _words(blk), index, len(blk), flags)
    return cv


def _subtree(data, first_chunk, root):
    if len(data) <= 1024:
        return _chunk_cv(data, first_chunk, root)
    n_chunks = (len(data) + 1023) // 1024
    left_chunks = 1 << ((n_chunks - 1).bit_length() - 1)
    left = _subtree(data[:left_chunks * 1024], first_chunk, False)
    right = _subtree(data[left_chunks * 1024:], first_chunk + left_chunks, False)
    return _compress(IV, left + right, 0, 64, PARENT | (ROOT if root else 0))


def blake3(data: bytes) -> bytes:
    return struct.pack("<8I", *_subtree(bytes(data), 0, True))
