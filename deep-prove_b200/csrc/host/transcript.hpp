// Host-side Fiat-Shamir transcript with the method names of the reference's
// `dp_crypto::arkyper::transcript::{Transcript, blake3::Blake3Transcript}`
// (zkml/src/lib.rs:106-108; append_scalars / append_and_sample /
// challenge_scalar as called in zkml/src/lookup/logup_gkr/prover.rs:163-173,
// 284-288).  The transcript stays on the host; only challenges cross to the GPU.
//
// The reference's byte format is defined in the dp-crypto crate, which is not
// part of the reference tree.  This implementation's format:
//   state_0    = BLAKE3("dpb-transcript-v1" || label)
//   absorb(t,m): state = BLAKE3(state || u32le(round) || u32le(|t|) || t || m); round += 1
//   append_scalars(v)    = absorb("scalars", u64le(|v|) || canonical bytes of each v)
//   append_and_sample(l) = absorb("label", l); challenge_scalar()
//   challenge_scalar()   = absorb("challenge", ""); 64 bytes = BLAKE3(state||0) || BLAKE3(state||1)
//        BN254 Fr        : the 64 bytes as a little-endian integer mod r
//        Goldilocks ext  : c0 = bytes[0:16] mod p, c1 = bytes[32:48] mod p
// Canonical bytes: Fr = 32-byte little-endian integer (ark_serialize's form);
// Goldilocks ext = c0 || c1, 8 bytes each.
#pragma once
#include <string>
#include <vector>

#include "../family.cuh"
#include "blake3.hpp"

namespace dpb {

// ---- canonical encodings and wide reduction per family ---------------------
inline void to_canonical(const Gl2& a, uint8_t* out) {
    memcpy(out, &a.c0, 8);
    memcpy(out + 8, &a.c1, 8);
}
inline void to_canonical(const Fr& a, uint8_t* out) {
    const Fr c = fr_from_mont(a);
    memcpy(out, c.l, 32);
}
inline size_t canonical_size(const Gl2&) { return 16; }
inline size_t canonical_size(const Fr&) { return 32; }

inline void challenge_from_bytes(const uint8_t b[64], Gl2* out) {
    uint64_t w[2];
    memcpy(w, b, 16);
    out->c0 = gl_reduce128(w[0], w[1]);
    memcpy(w, b + 32, 16);
    out->c1 = gl_reduce128(w[0], w[1]);
}
inline void challenge_from_bytes(const uint8_t b[64], Fr* out) {
    // value = lo + hi * 2^256 (mod r), lo and hi 256-bit little-endian integers
    Fr part[2];
    for (int h = 0; h < 2; h++) {
        memcpy(part[h].l, b + 32 * h, 32);
        // bring below r: 2^256 / r < 6
        for (int i = 0; i < 6; i++) {
            uint64_t bw = 0;
            Fr d;
            d.l[0] = sbb(part[h].l[0], DPB_FR_P0, bw);
            d.l[1] = sbb(part[h].l[1], DPB_FR_P1, bw);
            d.l[2] = sbb(part[h].l[2], DPB_FR_P2, bw);
            d.l[3] = sbb(part[h].l[3], DPB_FR_P3, bw);
            if (bw) break;
            part[h] = d;
        }
        part[h] = fr_to_mont(part[h]);
    }
    // Montgomery form of 2^256 mod r is R*R mod r
    *out = fr_add(part[0], fr_mul(part[1], fr_rr()));
}

template <class F>
class Blake3Transcript {
   public:
    typedef typename F::E E;

    explicit Blake3Transcript(const void* label, size_t len) {
        std::vector<uint8_t> m;
        static const char kDomain[] = "dpb-transcript-v1";
        m.insert(m.end(), kDomain, kDomain + sizeof(kDomain) - 1);
        m.insert(m.end(), (const uint8_t*)label, (const uint8_t*)label + len);
        blake3::hash(m.data(), m.size(), state_);
        round_ = 0;
    }

    void append_scalars(const E* v, size_t n) {
        std::vector<uint8_t> m(8 + n * canonical_size(E()));
        const uint64_t n64 = n;
        memcpy(m.data(), &n64, 8);
        for (size_t i = 0; i < n; i++) to_canonical(v[i], m.data() + 8 + i * canonical_size(E()));
        absorb("scalars", m.data(), m.size());
    }
    void append_scalars(const std::vector<E>& v) { append_scalars(v.data(), v.size()); }

    E challenge_scalar() {
        absorb("challenge", nullptr, 0);
        uint8_t in[33], out[64];
        memcpy(in, state_, 32);
        in[32] = 0;
        blake3::hash(in, 33, out);
        in[32] = 1;
        blake3::hash(in, 33, out + 32);
        E c;
        challenge_from_bytes(out, &c);
        return c;
    }

    E append_and_sample(const void* label, size_t len) {
        absorb("label", (const uint8_t*)label, len);
        return challenge_scalar();
    }
    E append_and_sample(const char* label) { return append_and_sample(label, strlen(label)); }

    // zkml/src/lib.rs:176-184
    std::vector<E> read_challenges(size_t n) {
        std::vector<E> out(n);
        for (size_t i = 0; i < n; i++) out[i] = challenge_scalar();
        return out;
    }

    const uint8_t* state() const { return state_; }
    uint32_t round() const { return round_; }

   private:
    void absorb(const char* tag, const uint8_t* msg, size_t len) {
        const uint32_t tl = (uint32_t)strlen(tag);
        std::vector<uint8_t> m(32 + 4 + 4 + tl + len);
        memcpy(m.data(), state_, 32);
        memcpy(m.data() + 32, &round_, 4);
        memcpy(m.data() + 36, &tl, 4);
        memcpy(m.data() + 40, tag, tl);
        if (len) memcpy(m.data() + 40 + tl, msg, len);
        blake3::hash(m.data(), m.size(), state_);
        round_++;
    }
    uint8_t state_[32];
    uint32_t round_;
};

}  // namespace dpb
