// Wire format of the host transport (control plane and CPU-tensor data plane).
//
// Every frame is a packed little-endian 24-byte header followed by
// `payload_bytes` of payload:
//   u16 version | u8 op | u8 flags | u32 seq | u32 tid | u32 chunk_index |
//   u32 payload_bytes | u32 crc
// `seq` is the process group's collective sequence number, `tid` distinguishes
// the messages of one collective (or carries the user tag of send/recv), and a
// payload larger than the transport's chunk size travels as consecutive frames
// with increasing `chunk_index` (the last one has FLAG_LAST_CHUNK).  `crc` is
// the ISO-3309 CRC-32 of the payload when FLAG_HAS_CRC is set, else 0.
// The handshake payload is 74 packed bytes: u16 version, u32 rank,
// u32 world_size, char hostname[64].
// Parity: reference csrc/transport/Protocol.hpp:14-168 (same sizes, same op
// codes, same CRC polynomial; check value of "123456789" is 0xCBF43926).
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <cstring>

#include "common/version.h"

namespace mccl {

enum class OpType : uint8_t {
  ALLREDUCE = 1,
  BROADCAST = 2,
  BARRIER = 3,
  ALLGATHER = 4,
  REDUCE_SCATTER = 5,
  SEND = 6,
  RECV = 7,
  HANDSHAKE = 10,
  HEARTBEAT = 11,
  ABORT = 255,
};

enum MsgFlags : uint8_t {
  FLAG_NONE = 0,
  FLAG_HAS_CRC = 1 << 0,
  FLAG_LAST_CHUNK = 1 << 1,
  FLAG_COMPRESSED = 1 << 2,
  FLAG_GOODBYE = 1 << 3,  // on a HEARTBEAT frame: the sender is shutting down in an orderly way
};

#pragma pack(push, 1)
struct MessageHeader {
  uint16_t version;
  uint8_t op;
  uint8_t flags;
  uint32_t seq;
  uint32_t tid;
  uint32_t chunk_index;
  uint32_t payload_bytes;
  uint32_t crc;
};

struct HandshakePayload {
  uint16_t version;
  uint32_t rank;
  uint32_t world_size;
  char hostname[64];
};
#pragma pack(pop)

static_assert(sizeof(MessageHeader) == 24, "frame header must be 24 bytes");
static_assert(sizeof(HandshakePayload) == 74, "handshake payload must be 74 bytes");
#if defined(__BYTE_ORDER__) && defined(__ORDER_LITTLE_ENDIAN__)
static_assert(__BYTE_ORDER__ == __ORDER_LITTLE_ENDIAN__, "wire format is little-endian");
#endif

inline MessageHeader make_header(OpType op, uint32_t seq, uint32_t tid, uint32_t chunk_index,
                                 uint32_t payload_bytes, uint8_t flags = 0, uint32_t crc = 0) {
  MessageHeader h;
  h.version = MCCL_PROTOCOL_VERSION;
  h.op = static_cast<uint8_t>(op);
  h.flags = flags;
  h.seq = seq;
  h.tid = tid;
  h.chunk_index = chunk_index;
  h.payload_bytes = payload_bytes;
  h.crc = crc;
  return h;
}

// CRC-32 (ISO 3309 / zlib polynomial 0xEDB88320, reflected), slicing-by-8.
namespace crc_detail {
struct Tables {
  uint32_t t[8][256];
  Tables() {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
      t[0][i] = c;
    }
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = t[0][i];
      for (int s = 1; s < 8; ++s) {
        c = t[0][c & 0xFF] ^ (c >> 8);
        t[s][i] = c;
      }
    }
  }
};
inline const Tables& tables() {
  static const Tables tb;
  return tb;
}
}  // namespace crc_detail

inline uint32_t crc32_update(uint32_t crc, const void* data, size_t n) {
  const auto& T = crc_detail::tables().t;
  const uint8_t* p = static_cast<const uint8_t*>(data);
  uint32_t c = ~crc;
  while (n && (reinterpret_cast<uintptr_t>(p) & 7)) {
    c = T[0][(c ^ *p++) & 0xFF] ^ (c >> 8);
    --n;
  }
  while (n >= 8) {
    uint64_t w;
    std::memcpy(&w, p, 8);
    uint32_t lo = static_cast<uint32_t>(w) ^ c;
    uint32_t hi = static_cast<uint32_t>(w >> 32);
    c = T[7][lo & 0xFF] ^ T[6][(lo >> 8) & 0xFF] ^ T[5][(lo >> 16) & 0xFF] ^ T[4][lo >> 24] ^
        T[3][hi & 0xFF] ^ T[2][(hi >> 8) & 0xFF] ^ T[1][(hi >> 16) & 0xFF] ^ T[0][hi >> 24];
    p += 8;
    n -= 8;
  }
  while (n--) c = T[0][(c ^ *p++) & 0xFF] ^ (c >> 8);
  return ~c;
}

inline uint32_t crc32_compute(const void* data, size_t n) { return crc32_update(0, data, n); }

}  // namespace mccl
