// Snappy block format, written from the public format description (no library is linked).
//
// The reference compresses RPC bodies between worker and server and between servers with Snappy
// (kraken/common/compress.h:18-91: SnappySink / SnappySource around snappy::Compress and
// snappy::Uncompress; header byte CompressType::kSnappy = 1, kraken/rpc/protocol.h:7-10).  The TCP
// deployment of this framework writes the same byte stream for code 1, so a body produced here is
// readable by any Snappy decoder and the other way round.
//
// Stream = uncompressed length as little-endian base-128 varint, then elements.  The low two bits of
// an element's first byte give its kind:
//   00 literal: (length - 1) in the upper six bits, or 60..63 = 1..4 little-endian length bytes follow;
//   01 copy, 11-bit offset: length 4..11 in bits 2..4, offset bits 8..10 in bits 5..7, low offset byte follows;
//   10 copy, 16-bit offset: (length - 1) in the upper six bits, two offset bytes follow;
//   11 copy, 32-bit offset: (length - 1) in the upper six bits, four offset bytes follow.
// The compressor works on independent 64 KiB blocks with a 2^14-entry hash table of 4-byte windows,
// so offsets fit 16 bits and kind 11 is only ever read.
#pragma once

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace kb {
namespace snappy_codec {

namespace detail {

constexpr size_t kBlockBytes = 1u << 16;
constexpr int kTableBits = 14;

inline uint32_t Read32(const char* p) {
  uint32_t v;
  std::memcpy(&v, p, sizeof(v));
  return v;
}
inline uint64_t Read64(const char* p) {
  uint64_t v;
  std::memcpy(&v, p, sizeof(v));
  return v;
}
inline uint32_t Bucket(uint32_t window) { return (window * 0x1e35a7bdu) >> (32 - kTableBits); }

inline void EmitLiteral(std::string* out, const char* src, size_t len) {
  if (len == 0) return;
  const size_t n = len - 1;
  if (n < 60) {
    out->push_back(static_cast<char>(n << 2));
  } else {
    const int extra = n < (1u << 8) ? 1 : n < (1u << 16) ? 2 : n < (1u << 24) ? 3 : 4;
    out->push_back(static_cast<char>((59 + extra) << 2));
    for (int b = 0; b < extra; ++b) out->push_back(static_cast<char>((n >> (8 * b)) & 0xff));
  }
  out->append(src, len);
}

inline void EmitOneCopy(std::string* out, size_t offset, size_t len) {  // len in 1..64
  if (len >= 4 && len <= 11 && offset < 2048) {
    out->push_back(static_cast<char>(1 | ((len - 4) << 2) | ((offset >> 8) << 5)));
    out->push_back(static_cast<char>(offset & 0xff));
  } else {
    out->push_back(static_cast<char>(2 | ((len - 1) << 2)));
    out->push_back(static_cast<char>(offset & 0xff));
    out->push_back(static_cast<char>((offset >> 8) & 0xff));
  }
}

inline void EmitCopy(std::string* out, size_t offset, size_t len) {
  // pieces of 64; a remainder of 1..3 after such a piece would need the long form, so the piece
  // before a short tail is cut to 60
  while (len >= 68) {
    EmitOneCopy(out, offset, 64);
    len -= 64;
  }
  if (len > 64) {
    EmitOneCopy(out, offset, 60);
    len -= 60;
  }
  EmitOneCopy(out, offset, len);
}

inline void CompressBlock(const char* base, size_t n, std::string* out, uint16_t* table) {
  std::memset(table, 0, sizeof(uint16_t) << kTableBits);
  size_t pending = 0;  // start of the bytes not yet emitted
  if (n >= 16) {
    const size_t last_probe = n - 8;
    size_t pos = 1;
    uint32_t miss_credit = 32;  // the stride grows by 1/32 byte per miss: incompressible data is skipped fast
    while (pos <= last_probe) {
      const uint32_t window = Read32(base + pos);
      const uint32_t b = Bucket(window);
      const size_t cand = table[b];
      table[b] = static_cast<uint16_t>(pos);
      if (cand >= pos || Read32(base + cand) != window) {
        pos += miss_credit >> 5;
        ++miss_credit;
        continue;
      }
      EmitLiteral(out, base + pending, pos - pending);
      size_t len = 4;
      for (;;) {
        if (pos + len + 8 > n) {
          while (pos + len < n && base[pos + len] == base[cand + len]) ++len;
          break;
        }
        const uint64_t diff = Read64(base + pos + len) ^ Read64(base + cand + len);
        if (diff != 0) {
          len += static_cast<size_t>(__builtin_ctzll(diff)) >> 3;
          break;
        }
        len += 8;
      }
      EmitCopy(out, pos - cand, len);
      pos += len;
      pending = pos;
      miss_credit = 32;
      if (pos <= last_probe) table[Bucket(Read32(base + pos - 1))] = static_cast<uint16_t>(pos - 1);
    }
  }
  EmitLiteral(out, base + pending, n - pending);
}

}  // namespace detail

// Appends the Snappy stream of [data, data + n) to *out.
inline void Compress(const char* data, size_t n, std::string* out) {
  out->reserve(out->size() + 32 + n + n / 6);
  for (size_t v = n;;) {
    if (v < 128) {
      out->push_back(static_cast<char>(v));
      break;
    }
    out->push_back(static_cast<char>((v & 0x7f) | 0x80));
    v >>= 7;
  }
  std::vector<uint16_t> table(1u << detail::kTableBits);
  for (size_t at = 0; at < n; at += detail::kBlockBytes) {
    const size_t len = n - at < detail::kBlockBytes ? n - at : detail::kBlockBytes;
    detail::CompressBlock(data + at, len, out, table.data());
  }
}

// Decodes a Snappy stream into *out (replaced).  False on any malformed input: a truncated element,
// an offset that reaches before the start, or a length that disagrees with the header.
inline bool Uncompress(const char* data, size_t n, std::string* out) {
  const unsigned char* ip = reinterpret_cast<const unsigned char*>(data);
  const unsigned char* const end = ip + n;
  uint64_t total = 0;
  for (int shift = 0;; shift += 7) {
    if (ip >= end || shift > 35) return false;
    const unsigned char b = *ip++;
    total |= static_cast<uint64_t>(b & 0x7f) << shift;
    if (b < 128) break;
  }
  if (total > (1ull << 32)) return false;
  // the densest element is a 3-byte copy of 64 bytes: a stream cannot expand by more than ~21.4 x, so a header
  // that claims more is damaged (and must not make this side allocate gigabytes for a few bytes of input)
  if (total > 22ull * n + 64) return false;
  const size_t want = static_cast<size_t>(total);
  out->assign(want, '\0');
  char* dst = want ? &(*out)[0] : nullptr;
  size_t op = 0;
  while (ip < end) {
    const unsigned tag = *ip++;
    const unsigned kind = tag & 3;
    if (kind == 0) {
      size_t len = (tag >> 2) + 1;
      if (len > 60) {
        const size_t extra = len - 60;
        if (static_cast<size_t>(end - ip) < extra) return false;
        size_t v = 0;
        for (size_t b = 0; b < extra; ++b) v |= static_cast<size_t>(ip[b]) << (8 * b);
        ip += extra;
        len = v + 1;
      }
      if (len > static_cast<size_t>(end - ip) || len > want - op) return false;
      std::memcpy(dst + op, ip, len);
      ip += len;
      op += len;
      continue;
    }
    size_t len, offset;
    const size_t tail = kind == 1 ? 1 : kind == 2 ? 2 : 4;
    if (static_cast<size_t>(end - ip) < tail) return false;
    if (kind == 1) {
      len = ((tag >> 2) & 7) + 4;
      offset = (static_cast<size_t>(tag >> 5) << 8) | ip[0];
    } else {
      len = (tag >> 2) + 1;
      offset = 0;
      for (size_t b = 0; b < tail; ++b) offset |= static_cast<size_t>(ip[b]) << (8 * b);
    }
    ip += tail;
    if (offset == 0 || offset > op || len > want - op) return false;
    if (offset >= len) {
      std::memcpy(dst + op, dst + op - offset, len);
    } else {
      for (size_t k = 0; k < len; ++k) dst[op + k] = dst[op + k - offset];  // overlapping copy = a run
    }
    op += len;
  }
  return op == want;
}

}  // namespace snappy_codec
}  // namespace kb
