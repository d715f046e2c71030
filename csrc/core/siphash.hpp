// Streaming SipHash with configurable rounds. SipHasher13 with a zero key is the function behind
// Rust's `std::collections::hash_map::DefaultHasher`, which the reference uses for predictor and
// checkpoint state hashes (nangila-core/src/predictor.rs:455-477, checkpoint.rs:57-85,
// fixed_point.rs:312-319). Integers are fed as their little-endian bytes, `usize` as 8 bytes.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace nangila {

template <int C_ROUNDS, int D_ROUNDS>
class SipHasher {
 public:
  explicit SipHasher(uint64_t k0 = 0, uint64_t k1 = 0) {
    v0_ = k0 ^ 0x736f6d6570736575ull;
    v1_ = k1 ^ 0x646f72616e646f6dull;
    v2_ = k0 ^ 0x6c7967656e657261ull;
    v3_ = k1 ^ 0x7465646279746573ull;
  }

  void write(const void* data, size_t len) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    length_ += len;
    if (ntail_ != 0) {
      while (len > 0 && ntail_ < 8) {
        tail_ |= uint64_t(*p) << (8 * ntail_);
        ++ntail_;
        ++p;
        --len;
      }
      if (ntail_ < 8) return;
      compress(tail_);
      tail_ = 0;
      ntail_ = 0;
    }
    while (len >= 8) {
      uint64_t m;
      std::memcpy(&m, p, 8);  // little-endian host assumed
      compress(m);
      p += 8;
      len -= 8;
    }
    while (len > 0) {
      tail_ |= uint64_t(*p) << (8 * ntail_);
      ++ntail_;
      ++p;
      --len;
    }
  }
  void write_u8(uint8_t v) { write(&v, 1); }
  void write_u32(uint32_t v) { write(&v, 4); }
  void write_i32(int32_t v) { write(&v, 4); }
  void write_u64(uint64_t v) { write(&v, 8); }
  void write_usize(size_t v) { write_u64(static_cast<uint64_t>(v)); }

  uint64_t finish() const {
    uint64_t v0 = v0_, v1 = v1_, v2 = v2_, v3 = v3_;
    uint64_t b = (uint64_t(length_ & 0xff) << 56) | tail_;
    v3 ^= b;
    for (int i = 0; i < C_ROUNDS; ++i) round(v0, v1, v2, v3);
    v0 ^= b;
    v2 ^= 0xff;
    for (int i = 0; i < D_ROUNDS; ++i) round(v0, v1, v2, v3);
    return v0 ^ v1 ^ v2 ^ v3;
  }

 private:
  static uint64_t rotl(uint64_t x, int b) { return (x << b) | (x >> (64 - b)); }
  static void round(uint64_t& v0, uint64_t& v1, uint64_t& v2, uint64_t& v3) {
    v0 += v1; v1 = rotl(v1, 13); v1 ^= v0; v0 = rotl(v0, 32);
    v2 += v3; v3 = rotl(v3, 16); v3 ^= v2;
    v0 += v3; v3 = rotl(v3, 21); v3 ^= v0;
    v2 += v1; v1 = rotl(v1, 17); v1 ^= v2; v2 = rotl(v2, 32);
  }
  void compress(uint64_t m) {
    v3_ ^= m;
    for (int i = 0; i < C_ROUNDS; ++i) round(v0_, v1_, v2_, v3_);
    v0_ ^= m;
  }
  uint64_t v0_, v1_, v2_, v3_;
  uint64_t tail_ = 0;
  size_t ntail_ = 0;
  size_t length_ = 0;
};

using SipHasher13 = SipHasher<1, 3>;
using SipHasher24 = SipHasher<2, 4>;

}  // namespace nangila
