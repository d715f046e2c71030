// Wire packet: 32-byte little-endian header + payload, protected by an IEEE CRC32 of the payload.
// Used by the CPU/gloo transport, by the C ABI and for integrity checks of staging buffers.
//
// Parity: nangila-core/src/packet.rs:10-31 (magic "NG" 0x4E47, version 1, flag bits), :47-68 and
// :182-238 (header layout and (de)serialisation), :241-274 (table CRC32, polynomial 0xEDB88320),
// :278-314 (Packet new/verify/to_bytes/from_bytes).
#pragma once
#include <array>
#include <cstdint>
#include <cstring>
#include <optional>
#include <vector>

namespace nangila {

constexpr uint16_t kPacketMagic = 0x4E47;
constexpr uint8_t kProtocolVersion = 1;

namespace flags {
constexpr uint8_t FORCE_SYNC = 0x01;
constexpr uint8_t DRIVER = 0x02;
constexpr uint8_t PASSENGER = 0x04;
constexpr uint8_t ACK_REQUEST = 0x08;
constexpr uint8_t ACK_RESPONSE = 0x10;
constexpr uint8_t DESYNC_RECOVERY = 0x20;
constexpr uint8_t PARTIAL_RETRANSMIT = 0x40;
// Addition to the reference's flag set: the sender quantized the raw gradient (plus error feedback)
// without subtracting a prediction, so the receiver must not add one.
constexpr uint8_t NO_PREDICTION = 0x80;
}  // namespace flags

namespace detail {
// Slicing-by-8 tables: row 0 is the classic byte table; row k advances a byte that lies k positions
// further from the end of an 8-byte group, so eight bytes are folded per step.
inline const std::array<std::array<uint32_t, 256>, 8>& crc32_tables() {
  static const std::array<std::array<uint32_t, 256>, 8> tables = [] {
    std::array<std::array<uint32_t, 256>, 8> t{};
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1u) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
      t[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; ++i)
      for (int k = 1; k < 8; ++k) t[k][i] = t[0][t[k - 1][i] & 0xff] ^ (t[k - 1][i] >> 8);
    return t;
  }();
  return tables;
}
inline const std::array<uint32_t, 256>& crc32_table() { return crc32_tables()[0]; }
template <class T>
inline void put_le(uint8_t* p, T v) {
  for (size_t i = 0; i < sizeof(T); ++i) p[i] = uint8_t((uint64_t(v) >> (8 * i)) & 0xff);
}
template <class T>
inline T get_le(const uint8_t* p) {
  uint64_t v = 0;
  for (size_t i = 0; i < sizeof(T); ++i) v |= uint64_t(p[i]) << (8 * i);
  return static_cast<T>(v);
}
}  // namespace detail

// Incremental form: pass the previous return value as `crc` to continue over a second buffer.
inline uint32_t crc32_update(uint32_t crc, const uint8_t* data, size_t len) {
  const auto& T = detail::crc32_tables();
  const auto& t = T[0];
  uint32_t c = crc ^ 0xFFFFFFFFu;
  size_t i = 0;
  for (; i + 8 <= len; i += 8) {
    const uint32_t lo = c ^ (uint32_t(data[i]) | uint32_t(data[i + 1]) << 8 | uint32_t(data[i + 2]) << 16 |
                             uint32_t(data[i + 3]) << 24);
    c = T[7][lo & 0xff] ^ T[6][(lo >> 8) & 0xff] ^ T[5][(lo >> 16) & 0xff] ^ T[4][lo >> 24] ^ T[3][data[i + 4]] ^
        T[2][data[i + 5]] ^ T[1][data[i + 6]] ^ T[0][data[i + 7]];
  }
  for (; i < len; ++i) c = t[(c ^ data[i]) & 0xff] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}
inline uint32_t compute_crc32(const uint8_t* data, size_t len) { return crc32_update(0, data, len); }
inline uint32_t compute_crc32(const std::vector<uint8_t>& v) { return compute_crc32(v.data(), v.size()); }
inline bool verify_crc32(const uint8_t* data, size_t len, uint32_t expected) {
  return compute_crc32(data, len) == expected;
}

struct PacketHeader {
  static constexpr size_t SIZE = 32;

  uint16_t magic = kPacketMagic;
  uint8_t version = kProtocolVersion;
  uint8_t flags = flags::DRIVER;
  uint32_t step = 0;
  uint32_t layer_id = 0;
  uint32_t crc32 = 0;
  uint64_t predictor_hash = 0;
  uint32_t start_offset = 0;
  uint32_t end_offset = 0;

  static PacketHeader with_flags(uint8_t f, uint32_t step, uint32_t layer) {
    PacketHeader h;
    h.flags = f;
    h.step = step;
    h.layer_id = layer;
    return h;
  }
  static PacketHeader new_driver(uint32_t step, uint32_t layer) { return with_flags(flags::DRIVER, step, layer); }
  static PacketHeader new_passenger(uint32_t step, uint32_t layer) { return with_flags(flags::PASSENGER, step, layer); }
  static PacketHeader new_force_sync(uint32_t step, uint32_t layer) {
    return with_flags(flags::FORCE_SYNC | flags::DRIVER, step, layer);
  }
  static PacketHeader new_partial_retransmit(uint32_t step, uint32_t layer, uint32_t start, uint32_t end) {
    PacketHeader h = with_flags(flags::PARTIAL_RETRANSMIT | flags::DRIVER, step, layer);
    h.start_offset = start;
    h.end_offset = end;
    return h;
  }

  bool is_valid() const { return magic == kPacketMagic && version == kProtocolVersion; }
  bool is_force_sync() const { return flags & flags::FORCE_SYNC; }
  bool is_driver() const { return flags & flags::DRIVER; }
  bool is_passenger() const { return flags & flags::PASSENGER; }
  bool is_desync_recovery() const { return flags & flags::DESYNC_RECOVERY; }
  bool is_partial_retransmit() const { return flags & flags::PARTIAL_RETRANSMIT; }

  std::array<uint8_t, SIZE> to_bytes() const {
    std::array<uint8_t, SIZE> b{};
    detail::put_le<uint16_t>(&b[0], magic);
    b[2] = version;
    b[3] = flags;
    detail::put_le<uint32_t>(&b[4], step);
    detail::put_le<uint32_t>(&b[8], layer_id);
    detail::put_le<uint32_t>(&b[12], crc32);
    detail::put_le<uint64_t>(&b[16], predictor_hash);
    detail::put_le<uint32_t>(&b[24], start_offset);
    detail::put_le<uint32_t>(&b[28], end_offset);
    return b;
  }
  static std::optional<PacketHeader> from_bytes(const uint8_t* b, size_t len) {
    if (len < SIZE) return std::nullopt;
    PacketHeader h;
    h.magic = detail::get_le<uint16_t>(&b[0]);
    h.version = b[2];
    h.flags = b[3];
    h.step = detail::get_le<uint32_t>(&b[4]);
    h.layer_id = detail::get_le<uint32_t>(&b[8]);
    h.crc32 = detail::get_le<uint32_t>(&b[12]);
    h.predictor_hash = detail::get_le<uint64_t>(&b[16]);
    h.start_offset = detail::get_le<uint32_t>(&b[24]);
    h.end_offset = detail::get_le<uint32_t>(&b[28]);
    return h;
  }
  bool operator==(const PacketHeader& o) const {
    return magic == o.magic && version == o.version && flags == o.flags && step == o.step &&
           layer_id == o.layer_id && crc32 == o.crc32 && predictor_hash == o.predictor_hash &&
           start_offset == o.start_offset && end_offset == o.end_offset;
  }
};

struct Packet {
  PacketHeader header;
  std::vector<uint8_t> payload;

  Packet() = default;
  // Fills in the CRC of `payload`.
  Packet(PacketHeader h, std::vector<uint8_t> p) : header(h), payload(std::move(p)) {
    header.crc32 = compute_crc32(payload);
  }
  bool verify() const { return header.is_valid() && compute_crc32(payload) == header.crc32; }
  std::vector<uint8_t> to_bytes() const {
    std::vector<uint8_t> out(PacketHeader::SIZE + payload.size());
    auto h = header.to_bytes();
    std::memcpy(out.data(), h.data(), PacketHeader::SIZE);
    if (!payload.empty()) std::memcpy(out.data() + PacketHeader::SIZE, payload.data(), payload.size());
    return out;
  }
  static std::optional<Packet> from_bytes(const uint8_t* b, size_t len) {
    auto h = PacketHeader::from_bytes(b, len);
    if (!h) return std::nullopt;
    Packet p;
    p.header = *h;  // keep the transmitted CRC; verify() recomputes
    p.payload.assign(b + PacketHeader::SIZE, b + len);
    return p;
  }
};

}  // namespace nangila
