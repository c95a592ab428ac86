// Offline stand-in for the snappy library (see snappy.h).  Format facts used (public format
// description): a stream is the uncompressed length as a little-endian base-128 varint followed by
// elements whose first byte's low two bits give the kind: 00 literal (length-1 in the upper six bits, or
// 60..63 meaning that 1..4 length bytes follow), 01 copy with an 11-bit offset and length 4..11,
// 10 copy with a 16-bit offset and length 1..64, 11 copy with a 32-bit offset.
#include "snappy.h"

#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

namespace snappy {

Sink::~Sink() {}
char* Sink::GetAppendBuffer(size_t, char* scratch) { return scratch; }
void Sink::AppendAndTakeOwnership(char* bytes, size_t n, void (*deleter)(void*, const char*, size_t),
                                  void* deleter_arg) {
  Append(bytes, n);
  (*deleter)(deleter_arg, bytes, n);
}
char* Sink::GetAppendBufferVariable(size_t, size_t, char* scratch, size_t scratch_size, size_t* allocated_size) {
  *allocated_size = scratch_size;
  return scratch;
}
Source::~Source() {}

size_t MaxCompressedLength(size_t n) { return 32 + n + n / 6; }

namespace {

constexpr size_t kBlock = 1 << 16;
constexpr int kHashBits = 14;

inline uint32_t Load32(const char* p) {
  uint32_t v;
  memcpy(&v, p, 4);
  return v;
}
inline uint64_t Load64(const char* p) {
  uint64_t v;
  memcpy(&v, p, 8);
  return v;
}
inline uint32_t HashOf(uint32_t v) { return (v * 0x9E3779B1u) >> (32 - kHashBits); }

char* PutLiteral(char* op, const char* src, size_t len) {
  if (len == 0) return op;
  const size_t n = len - 1;
  if (n < 60) {
    *op++ = static_cast<char>(n << 2);
  } else {
    int bytes = n < (1u << 8) ? 1 : n < (1u << 16) ? 2 : n < (1u << 24) ? 3 : 4;
    *op++ = static_cast<char>((59 + bytes) << 2);
    for (int b = 0; b < bytes; ++b) *op++ = static_cast<char>((n >> (8 * b)) & 0xff);
  }
  memcpy(op, src, len);
  return op + len;
}

char* PutCopyUpTo64(char* op, size_t offset, size_t len) {
  if (len >= 4 && len < 12 && offset < 2048) {
    *op++ = static_cast<char>(1 | ((len - 4) << 2) | ((offset >> 8) << 5));
    *op++ = static_cast<char>(offset & 0xff);
  } else {
    *op++ = static_cast<char>(2 | ((len - 1) << 2));
    *op++ = static_cast<char>(offset & 0xff);
    *op++ = static_cast<char>((offset >> 8) & 0xff);
  }
  return op;
}

char* PutCopy(char* op, size_t offset, size_t len) {
  while (len >= 68) {
    op = PutCopyUpTo64(op, offset, 64);
    len -= 64;
  }
  if (len > 64) {
    op = PutCopyUpTo64(op, offset, 60);
    len -= 60;
  }
  return PutCopyUpTo64(op, offset, len);
}

// One block of at most 64 KiB; `table` has 1 << kHashBits entries.
char* CompressBlock(const char* base, size_t n, char* op, uint16_t* table) {
  memset(table, 0, sizeof(uint16_t) << kHashBits);
  size_t lit = 0;
  if (n >= 16) {
    const size_t limit = n - 8;  // positions at or below this can load 8 bytes
    size_t ip = 1;
    uint32_t skip = 32;
    while (ip <= limit) {
      const uint32_t cur = Load32(base + ip);
      const uint32_t h = HashOf(cur);
      const size_t cand = table[h];
      table[h] = static_cast<uint16_t>(ip);
      if (cand < ip && Load32(base + cand) == cur) {
        op = PutLiteral(op, base + lit, ip - lit);
        size_t len = 4;
        while (ip + len + 8 <= n) {
          const uint64_t x = Load64(base + ip + len) ^ Load64(base + cand + len);
          if (x != 0) {
            len += static_cast<size_t>(__builtin_ctzll(x)) >> 3;
            goto matched;
          }
          len += 8;
        }
        while (ip + len < n && base[ip + len] == base[cand + len]) ++len;
      matched:
        op = PutCopy(op, ip - cand, len);
        ip += len;
        lit = ip;
        skip = 32;
        if (ip <= limit && ip >= 1) table[HashOf(Load32(base + ip - 1))] = static_cast<uint16_t>(ip - 1);
      } else {
        ip += skip >> 5;  // strides grow over data that does not match, as snappy's do
        ++skip;
      }
    }
  }
  return PutLiteral(op, base + lit, n - lit);
}

}  // namespace

size_t Compress(Source* reader, Sink* writer) {
  size_t remaining = reader->Available();
  size_t written = 0;
  char head[10];
  int hn = 0;
  for (size_t v = remaining; ; ) {
    if (v < 128) {
      head[hn++] = static_cast<char>(v);
      break;
    }
    head[hn++] = static_cast<char>((v & 0x7f) | 0x80);
    v >>= 7;
  }
  writer->Append(head, hn);
  written += hn;

  std::vector<uint16_t> table(1u << kHashBits);
  std::vector<char> gather;
  std::vector<char> outbuf(MaxCompressedLength(kBlock));
  while (remaining > 0) {
    const size_t want = remaining < kBlock ? remaining : kBlock;
    size_t frag = 0;
    const char* p = reader->Peek(&frag);
    size_t consumed_from_reader = 0;
    if (frag < want) {  // the source hands out pieces smaller than a block: assemble one
      gather.resize(want);
      size_t have = 0;
      while (have < want) {
        p = reader->Peek(&frag);
        if (frag == 0) return 0;
        const size_t take = frag < want - have ? frag : want - have;
        memcpy(gather.data() + have, p, take);
        reader->Skip(take);
        have += take;
      }
      p = gather.data();
    } else {
      consumed_from_reader = want;
    }
    char* dst = writer->GetAppendBuffer(outbuf.size(), outbuf.data());
    char* end = CompressBlock(p, want, dst, table.data());
    writer->Append(dst, static_cast<size_t>(end - dst));
    written += static_cast<size_t>(end - dst);
    if (consumed_from_reader) reader->Skip(consumed_from_reader);
    remaining -= want;
  }
  return written;
}

bool Uncompress(Source* compressed, Sink* uncompressed) {
  // gather the stream (the reference's sources hand out everything in one piece)
  size_t avail = compressed->Available();
  size_t frag = 0;
  const char* in = compressed->Peek(&frag);
  std::vector<char> joined;
  if (frag < avail) {
    joined.reserve(avail);
    while (compressed->Available() > 0) {
      in = compressed->Peek(&frag);
      if (frag == 0) return false;
      joined.insert(joined.end(), in, in + frag);
      compressed->Skip(frag);
    }
    in = joined.data();
    avail = joined.size();
  }
  const unsigned char* ip = reinterpret_cast<const unsigned char*>(in);
  const unsigned char* const iend = ip + avail;

  uint64_t total = 0;
  int shift = 0;
  for (;;) {
    if (ip >= iend || shift > 28) return false;
    const unsigned char b = *ip++;
    total |= static_cast<uint64_t>(b & 0x7f) << shift;
    if (b < 128) break;
    shift += 7;
  }
  const size_t n = static_cast<size_t>(total);

  size_t got = 0;
  char* out = n ? uncompressed->GetAppendBufferVariable(n, n, nullptr, 0, &got) : nullptr;
  char* own = nullptr;
  if (n && (out == nullptr || got < n)) out = own = static_cast<char*>(malloc(n));
  size_t op = 0;
  bool ok = true;
  while (ip < iend && ok) {
    const unsigned tag = *ip++;
    const unsigned kind = tag & 3;
    if (kind == 0) {
      size_t len = (tag >> 2) + 1;
      if (len > 60) {
        const int bytes = static_cast<int>(len) - 60;
        if (ip + bytes > iend) { ok = false; break; }
        size_t v = 0;
        for (int b = 0; b < bytes; ++b) v |= static_cast<size_t>(ip[b]) << (8 * b);
        ip += bytes;
        len = v + 1;
      }
      if (len > static_cast<size_t>(iend - ip) || len > n - op) { ok = false; break; }
      memcpy(out + op, ip, len);
      ip += len;
      op += len;
    } else {
      size_t len, offset;
      if (kind == 1) {
        if (ip + 1 > iend) { ok = false; break; }
        len = ((tag >> 2) & 7) + 4;
        offset = (static_cast<size_t>(tag >> 5) << 8) | ip[0];
        ip += 1;
      } else if (kind == 2) {
        if (ip + 2 > iend) { ok = false; break; }
        len = (tag >> 2) + 1;
        offset = ip[0] | (static_cast<size_t>(ip[1]) << 8);
        ip += 2;
      } else {
        if (ip + 4 > iend) { ok = false; break; }
        len = (tag >> 2) + 1;
        offset = ip[0] | (static_cast<size_t>(ip[1]) << 8) | (static_cast<size_t>(ip[2]) << 16) |
                 (static_cast<size_t>(ip[3]) << 24);
        ip += 4;
      }
      if (offset == 0 || offset > op || len > n - op) { ok = false; break; }
      if (offset >= len) {
        memcpy(out + op, out + op - offset, len);
      } else {
        for (size_t k = 0; k < len; ++k) out[op + k] = out[op + k - offset];  // overlapping: a run
      }
      op += len;
    }
  }
  ok = ok && op == n;
  if (ok && n) uncompressed->Append(out, n);
  if (own) free(own);
  compressed->Skip(compressed->Available());
  return ok;
}

}  // namespace snappy
