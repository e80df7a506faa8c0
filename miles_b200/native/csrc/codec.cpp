// Byte codecs of the native runtime: the XXH64 checksum and a delta codec for weight tensors.
//
// A published weight version differs from the previous one in the low mantissa bits of most elements and not at all in
// many (frozen or slowly moving parameters).  XOR against the base turns "unchanged" into zero bytes; splitting the bytes
// of each element into planes (all low bytes, then all high bytes, ...) groups the zeros of the sign / exponent plane into
// long runs; a zero-run-length code then stores a run as one varint.  One pass, no entropy stage: the encoder runs at
// memory speed, which is what a weight publisher that has to keep up with training needs (the reference's disk-delta
// path compresses with zstd and checks xxhash sums, miles/utils/disk_delta.py).
#include <stdint.h>
#include <string.h>

namespace {

constexpr uint64_t P1 = 0x9E3779B185EBCA87ull, P2 = 0xC2B2AE3D27D4EB4Full, P3 = 0x165667B19E3779F9ull, P4 = 0x85EBCA77C2B2AE63ull,
                   P5 = 0x27D4EB2F165667C5ull;

inline uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t rd64(const uint8_t* p) { uint64_t v; memcpy(&v, p, 8); return v; }
inline uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }
inline uint64_t round1(uint64_t acc, uint64_t in) { return rotl(acc + in * P2, 31) * P1; }
inline uint64_t merge(uint64_t h, uint64_t v) { return (h ^ round1(0, v)) * P1 + P4; }

inline int put_varint(uint8_t* out, uint64_t v) {
  int n = 0;
  while (v >= 0x80) { out[n++] = static_cast<uint8_t>(v) | 0x80; v >>= 7; }
  out[n++] = static_cast<uint8_t>(v);
  return n;
}
inline bool get_varint(const uint8_t*& p, const uint8_t* end, uint64_t& v) {
  v = 0;
  for (int shift = 0; p < end && shift < 64; shift += 7) {
    const uint8_t b = *p++;
    v |= static_cast<uint64_t>(b & 0x7F) << shift;
    if (!(b & 0x80)) return true;
  }
  return false;
}

constexpr uint8_t kMagic[4] = {'M', 'Z', 'R', '1'};

}  // namespace

extern "C" {

// XXH64 of `len` bytes (little-endian host).
uint64_t mbrt_xxh64(const void* data, uint64_t len, uint64_t seed) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  const uint8_t* const end = p + len;
  uint64_t h;
  if (len >= 32) {
    uint64_t v1 = seed + P1 + P2, v2 = seed + P2, v3 = seed, v4 = seed - P1;
    const uint8_t* const limit = end - 32;
    do {
      v1 = round1(v1, rd64(p));
      v2 = round1(v2, rd64(p + 8));
      v3 = round1(v3, rd64(p + 16));
      v4 = round1(v4, rd64(p + 24));
      p += 32;
    } while (p <= limit);
    h = rotl(v1, 1) + rotl(v2, 7) + rotl(v3, 12) + rotl(v4, 18);
    h = merge(h, v1);
    h = merge(h, v2);
    h = merge(h, v3);
    h = merge(h, v4);
  } else {
    h = seed + P5;
  }
  h += len;
  while (p + 8 <= end) {
    h ^= round1(0, rd64(p));
    h = rotl(h, 27) * P1 + P4;
    p += 8;
  }
  if (p + 4 <= end) {
    h ^= static_cast<uint64_t>(rd32(p)) * P1;
    h = rotl(h, 23) * P2 + P3;
    p += 4;
  }
  while (p < end) {
    h ^= (*p++) * P5;
    h = rotl(h, 11) * P1;
  }
  h ^= h >> 33;
  h *= P2;
  h ^= h >> 29;
  h *= P3;
  h ^= h >> 32;
  return h;
}

// Upper bound of the encoded size for `n` input bytes.
uint64_t mbrt_delta_bound(uint64_t n) { return n + n / 64 + 64; }

// cur XOR base (base may be null: plain planes) → planes → zero-run-length.  `elem` = bytes per element (1, 2, 4 or 8), `n`
// a multiple of it.  Returns the encoded size, or −1 when `cap` is too small or the arguments are inconsistent.
int64_t mbrt_delta_encode(const uint8_t* cur, const uint8_t* base, uint64_t n, int32_t elem, uint8_t* out, uint64_t cap) {
  if (elem < 1 || elem > 8 || n % static_cast<uint64_t>(elem) || cap < 16) return -1;
  uint8_t* o = out;
  uint8_t* const oend = out + cap;
  memcpy(o, kMagic, 4);
  o += 4;
  o += put_varint(o, n);
  *o++ = static_cast<uint8_t>(elem);
  const uint64_t count = n / elem;
  for (int plane = 0; plane < elem; ++plane) {
    uint64_t i = 0;
    while (i < count) {
      // zeros
      uint64_t z = i;
      while (z < count) {
        const uint64_t at = z * elem + plane;
        if ((cur[at] ^ (base ? base[at] : 0)) != 0) break;
        ++z;
      }
      // literals: up to the next run of at least 4 zeros (shorter runs cost more as a token than as bytes)
      uint64_t l = z, zeros = 0;
      while (l < count) {
        const uint64_t at = l * elem + plane;
        if ((cur[at] ^ (base ? base[at] : 0)) == 0) {
          if (++zeros == 4) { l -= 3; break; }
        } else {
          zeros = 0;
        }
        ++l;
      }
      if (l == count && zeros > 0 && zeros < 4) zeros = 0;      // trailing short run stays literal
      const uint64_t lit = l - z;
      if (o + 20 + lit > oend) return -1;
      o += put_varint(o, z - i);
      o += put_varint(o, lit);
      for (uint64_t k = z; k < l; ++k) {
        const uint64_t at = k * elem + plane;
        *o++ = cur[at] ^ (base ? base[at] : 0);
      }
      i = l;
    }
  }
  return o - out;
}

// Inverse of `mbrt_delta_encode`: writes `n` bytes to `out` (XORed onto `base` when given).  Returns n, or −1 on a
// malformed stream (nothing outside [out, out + n) is written).
int64_t mbrt_delta_decode(const uint8_t* enc, uint64_t enc_len, const uint8_t* base, uint8_t* out, uint64_t n) {
  const uint8_t* p = enc;
  const uint8_t* const end = enc + enc_len;
  if (enc_len < 6 || memcmp(p, kMagic, 4) != 0) return -1;
  p += 4;
  uint64_t total = 0;
  if (!get_varint(p, end, total) || total != n || p >= end) return -1;
  const int elem = *p++;
  if (elem < 1 || elem > 8 || n % static_cast<uint64_t>(elem)) return -1;
  const uint64_t count = n / elem;
  for (int plane = 0; plane < elem; ++plane) {
    uint64_t i = 0;
    while (i < count) {
      uint64_t z = 0, lit = 0;
      if (!get_varint(p, end, z) || !get_varint(p, end, lit)) return -1;
      if (z > count - i || lit > count - i - z || lit > static_cast<uint64_t>(end - p)) return -1;
      for (uint64_t k = 0; k < z; ++k) {
        const uint64_t at = (i + k) * elem + plane;
        out[at] = base ? base[at] : 0;
      }
      i += z;
      for (uint64_t k = 0; k < lit; ++k) {
        const uint64_t at = (i + k) * elem + plane;
        out[at] = p[k] ^ (base ? base[at] : 0);
      }
      p += lit;
      i += lit;
      if (z == 0 && lit == 0) return -1;      // no progress: malformed
    }
  }
  return static_cast<int64_t>(n);
}

}  // extern "C"
