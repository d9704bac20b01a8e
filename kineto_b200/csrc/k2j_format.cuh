// Text-formatting primitives of the Chrome-trace emitter.  Everything here is generic over a
// "sink" that either counts bytes (size pass) or writes them (emit pass), so the two passes cannot
// disagree.  The header also compiles as plain C++ (K2J_HD drops the CUDA qualifiers) so the
// integer / fixed-point / shortest-double routines can be exercised on a CPU without a GPU.
//
// Behaviour being matched (reference project paths):
//   integers            std::to_chars            libkineto/include/TypedMetadataJson.h:160-170
//   doubles             fmt::format("{}", v)     libkineto/include/TypedMetadataJson.h:172-178
//   "us.nnn" timestamps fmt "{}.{:03}"           libkineto/src/output_json.cpp:124-126
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define K2J_HD __device__ __forceinline__
#define K2J_TABLE_QUALIFIER static __device__ const
#define K2J_CONST_TABLE static __constant__ const
#define K2J_CONSTEXPR __host__ __device__ constexpr
#else
#define K2J_CONSTEXPR constexpr
#define K2J_HD inline
#define K2J_TABLE_QUALIFIER static const
#define K2J_CONST_TABLE static const
#endif

#include "k2j_pow10.h"

namespace k2j {

// ------------------------------------------------------------------------------------------------
// 128-bit helpers
// ------------------------------------------------------------------------------------------------
K2J_HD uint64_t umulhi64(uint64_t a, uint64_t b) {
#if defined(__CUDA_ARCH__)
  return __umul64hi(a, b);
#else
  return (uint64_t)(((unsigned __int128)a * b) >> 64);
#endif
}
K2J_HD int clz64(uint64_t v) {
#if defined(__CUDA_ARCH__)
  return __clzll((long long)v);
#else
  return v ? __builtin_clzll(v) : 64;
#endif
}
K2J_HD uint64_t dbits(double d) {
#if defined(__CUDA_ARCH__)
  return (uint64_t)__double_as_longlong(d);
#else
  uint64_t u; memcpy(&u, &d, 8); return u;
#endif
}

// ------------------------------------------------------------------------------------------------
// Compile-time packed literals
// ------------------------------------------------------------------------------------------------
template <int N>
struct Lit {
  uint32_t w[(N + 3) / 4 > 0 ? (N + 3) / 4 : 1];
  K2J_CONSTEXPR Lit(const char (&s)[N + 1]) : w{} {
    for (int i = 0; i < N; i++) w[i / 4] |= (uint32_t)(unsigned char)s[i] << (8 * (i % 4));
  }
};
#define K2J_LIT(sink, str)                          \
  do {                                              \
    constexpr ::k2j::Lit<sizeof(str) - 1> _l(str);  \
    (sink).template lit<sizeof(str) - 1>(_l);       \
  } while (0)

// ------------------------------------------------------------------------------------------------
// Sinks.  put(w, len) / put64(w, len): append the low `len` (1..4 / 0..8) bytes of w; bytes of w above
// `len` must be zero.
// ------------------------------------------------------------------------------------------------
struct CountSink {
  static constexpr bool kCounting = true;
  uint32_t n = 0;
  K2J_HD void put(uint32_t, int len) { n += (uint32_t)len; }
  K2J_HD void put64(uint64_t, uint32_t len) { n += len; }
  K2J_HD void skip(uint32_t len) { n += len; }
  template <int N> K2J_HD void lit(const Lit<N>&) { n += N; }
};

#if !defined(__CUDACC__)
#include <string>
struct StringSink {  // CPU test sink
  static constexpr bool kCounting = false;
  std::string s;
  void put(uint32_t w, int len) { for (int i = 0; i < len; i++) s += (char)((w >> (8 * i)) & 0xff); }
  void put64(uint64_t w, uint32_t len) { for (uint32_t i = 0; i < len; i++) s += (char)((w >> (8 * i)) & 0xff); }
  void skip(uint32_t) {}
  template <int N> void lit(const Lit<N>& l) {
    for (int i = 0; i < N; i++) s += (char)((l.w[i / 4] >> (8 * (i % 4))) & 0xff);
  }
};
#endif

template <class S> K2J_HD void put8(S& s, uint64_t a, int len) { s.put64(a, (uint32_t)len); }  // len 1..8, bytes above len zero
template <class S> K2J_HD void put_char(S& s, char c) { s.put((uint32_t)(unsigned char)c, 1); }

// ------------------------------------------------------------------------------------------------
// Integers
// ------------------------------------------------------------------------------------------------
K2J_CONST_TABLE uint64_t kPow10_64[20] = {
    1ull, 10ull, 100ull, 1000ull, 10000ull, 100000ull, 1000000ull, 10000000ull, 100000000ull,
    1000000000ull, 10000000000ull, 100000000000ull, 1000000000000ull, 10000000000000ull,
    100000000000000ull, 1000000000000000ull, 10000000000000000ull, 100000000000000000ull,
    1000000000000000000ull, 10000000000000000000ull};

// Number of decimal digits of v (1 for 0).
K2J_HD int ndigits64(uint64_t v) {
  const uint64_t w = v | 1;            // 0 prints as one digit; setting bit 0 never crosses a power of ten
  int b = 64 - clz64(w);               // bit length, 1..64
  int d = (b * 1233) >> 12;            // floor(b * log10(2)): the digit count or one less
  return d + (w >= kPow10_64[d] ? 1 : 0);
}

// x < 10^8 -> its 8 zero-padded ASCII digits, most significant digit in the low byte.
K2J_HD uint64_t ascii8(uint32_t x) {
  uint32_t hi = x / 10000u, lo = x - hi * 10000u;
  uint64_t v = (uint64_t)hi | ((uint64_t)lo << 32);              // two 4-digit groups
  uint64_t t = ((v * 5243ull) >> 19) & 0x0000007F0000007Full;    // /100 in each group
  v = t | ((v - t * 100ull) << 16);                              // four 2-digit groups
  t = ((v * 103ull) >> 10) & 0x000F000F000F000Full;              // /10 in each group
  v = t | ((v - t * 10ull) << 8);                                // eight digits
  return v | 0x3030303030303030ull;
}

template <class S> K2J_HD void put_small(S& s, uint32_t x) {  // x < 10^8, no padding
  int d = ndigits64(x);
  put8(s, ascii8(x) >> (8 * (8 - d)), d);
}
template <class S> K2J_HD void put_u64(S& s, uint64_t v) {
  if (S::kCounting) { s.skip((uint32_t)ndigits64(v)); return; }
  if (v < 100000000ull) { put_small(s, (uint32_t)v); return; }
  uint64_t hi = v / 100000000ull;
  uint32_t lo = (uint32_t)(v - hi * 100000000ull);
  if (hi < 100000000ull) {
    put_small(s, (uint32_t)hi);
  } else {
    uint64_t top = hi / 100000000ull;
    uint32_t mid = (uint32_t)(hi - top * 100000000ull);
    put_small(s, (uint32_t)top);
    put8(s, ascii8(mid), 8);
  }
  put8(s, ascii8(lo), 8);
}
template <class S> K2J_HD void put_i64(S& s, int64_t v) {
  if (v < 0) { put_char(s, '-'); put_u64(s, 0ull - (uint64_t)v); }
  else put_u64(s, (uint64_t)v);
}
// "{}.{:03}" of (ns / 1000, ns % 1000) for ns >= 0.
template <class S> K2J_HD void put_ts(S& s, int64_t ns) {
  uint64_t us = (uint64_t)ns / 1000ull;
  uint32_t fr = (uint32_t)((uint64_t)ns - us * 1000ull);
  put_u64(s, us);
  if (S::kCounting) { s.skip(4); return; }
  uint32_t a = fr / 100u, b = (fr / 10u) % 10u, c = fr % 10u;
  s.put(0x2Eu | ((0x30u + a) << 8) | ((0x30u + b) << 16) | ((0x30u + c) << 24), 4);
}

// ------------------------------------------------------------------------------------------------
// Shortest round-trip decimal of a finite positive double (Schubfach, R. Giulietti, "The
// Schubfach way to render doubles", 2020), written from the published algorithm.
// Returns the decimal significand (no trailing zeros) and sets *exp10 so that
// value = significand * 10^(*exp10).
// ------------------------------------------------------------------------------------------------
K2J_HD int floor_log2_pow10(int e) { return (e * 1741647) >> 19; }
K2J_HD int floor_log10_pow2(int e) { return (e * 1262611) >> 22; }
K2J_HD int floor_log10_three_quarters_pow2(int e) { return (e * 1262611 - 524031) >> 22; }

K2J_HD uint64_t round_to_odd(uint64_t ghi, uint64_t glo, uint64_t cp) {
  uint64_t xhi = umulhi64(glo, cp);
  uint64_t ylo = ghi * cp, yhi = umulhi64(ghi, cp);
  uint64_t y0 = ylo + xhi;
  uint64_t y1 = yhi + (y0 < xhi ? 1 : 0);
  return y1 | (y0 > 1 ? 1 : 0);
}

K2J_HD uint64_t shortest_decimal(uint64_t bits, int* exp10) {
  const uint64_t f = bits & 0x000FFFFFFFFFFFFFull;
  const int e = (int)((bits >> 52) & 0x7FF);
  uint64_t c; int q;
  if (e != 0) { c = f | 0x0010000000000000ull; q = e - 1075; } else { c = f; q = -1074; }
  const bool even = (c & 1) == 0;
  const bool lower_closer = (f == 0 && e > 1);
  const uint64_t cbl = 4 * c - 2 + (lower_closer ? 1 : 0);
  const uint64_t cb = 4 * c;
  const uint64_t cbr = 4 * c + 2;
  const int k = lower_closer ? floor_log10_three_quarters_pow2(q) : floor_log10_pow2(q);
  const int h = q + floor_log2_pow10(-k) + 1;
  const uint64_t ghi = k2j_pow10_tab[-k - K2J_POW10_MIN][0];
  const uint64_t glo = k2j_pow10_tab[-k - K2J_POW10_MIN][1];
  const uint64_t vbl = round_to_odd(ghi, glo, cbl << h);
  const uint64_t vb = round_to_odd(ghi, glo, cb << h);
  const uint64_t vbr = round_to_odd(ghi, glo, cbr << h);
  const uint64_t lower = vbl + (even ? 0 : 1);
  const uint64_t upper = vbr - (even ? 0 : 1);
  const uint64_t s = vb / 4;
  uint64_t dec; int ke = k;
  bool done = false;
  if (s >= 10) {
    const uint64_t sp = s / 10;
    const bool up_inside = lower <= 40 * sp;
    const bool wp_inside = 40 * sp + 40 <= upper;
    if (up_inside != wp_inside) { dec = sp + (wp_inside ? 1 : 0); ke = k + 1; done = true; }
  }
  if (!done) {
    const bool u_inside = lower <= 4 * s;
    const bool w_inside = 4 * s + 4 <= upper;
    if (u_inside != w_inside) dec = s + (w_inside ? 1 : 0);
    else {
      const uint64_t mid = 4 * s + 2;
      const bool round_up = vb > mid || (vb == mid && (s & 1) != 0);
      dec = s + (round_up ? 1 : 0);
    }
  }
  // strip trailing zeros
  while (true) {
    uint64_t qd = dec / 10;
    if (qd * 10 != dec || dec == 0) break;
    dec = qd; ke++;
  }
  *exp10 = ke;
  return dec;
}

// Length of fmt's default rendering of finite `v`, and the layout decisions shared by both passes.
struct DoubleLayout {
  uint64_t dec; int nd; int e10; bool neg; bool zero;
};
K2J_HD DoubleLayout double_layout(double v) {
  DoubleLayout L;
  uint64_t b = dbits(v);
  L.neg = (b >> 63) != 0;
  b &= 0x7FFFFFFFFFFFFFFFull;
  L.zero = (b == 0);
  if (L.zero) { L.dec = 0; L.nd = 1; L.e10 = 0; return L; }
  int k;
  L.dec = shortest_decimal(b, &k);
  L.nd = ndigits64(L.dec);
  L.e10 = k + L.nd - 1;
  return L;
}
K2J_HD bool double_is_finite(double v) { return ((dbits(v) >> 52) & 0x7FF) != 0x7FF; }

// Non-finite doubles print as nan / -nan / inf / -inf (the caller adds the quotes).
template <class S> K2J_HD void put_nonfinite(S& s, double v) {
  uint64_t b = dbits(v);
  if (b >> 63) put_char(s, '-');
  if (b & 0x000FFFFFFFFFFFFFull) s.put(0x006E616Eu, 3);  // "nan"
  else s.put(0x00666E69u, 3);                            // "inf"
}

// The 17 zero-padded decimal digits of dec (< 10^17) as ASCII in three registers: characters 0..7,
// 8..15 and 16.  Pieces of the digit string are then cut out with shifts, eight characters at a time.
struct Digits17 { uint64_t x0, x1, x2; };
K2J_HD Digits17 digits17(uint64_t dec) {
  const uint64_t hi = dec / 100000000ull;
  const uint32_t lo = (uint32_t)(dec - hi * 100000000ull);
  const uint32_t top = (uint32_t)(hi / 100000000ull);
  const uint32_t mid = (uint32_t)(hi - (uint64_t)top * 100000000ull);
  const uint64_t a1 = ascii8(mid), a2 = ascii8(lo);
  Digits17 D;
  D.x0 = (uint64_t)(0x30u + top) | (a1 << 8);
  D.x1 = (a1 >> 56) | (a2 << 8);
  D.x2 = a2 >> 56;
  return D;
}
// the 8 characters starting at character `o` (0..16); characters past the 17th read as zero bytes
K2J_HD uint64_t digits_at(const Digits17& D, int o) {
  const int wi = o >> 3, sh = (o & 7) * 8;
  const uint64_t a = wi == 0 ? D.x0 : wi == 1 ? D.x1 : D.x2;
  const uint64_t b = wi == 0 ? D.x1 : wi == 1 ? D.x2 : 0ull;
  return (a >> sh) | ((b << 1) << (63 - sh));
}
template <class S> K2J_HD void put_digits(S& s, const Digits17& D, int o, int n) {
  while (n > 0) {
    const int m = n < 8 ? n : 8;
    s.put64(digits_at(D, o) & (~0ull >> (8 * (8 - m))), (uint32_t)m);
    o += m; n -= m;
  }
}
template <class S> K2J_HD void put_zeros(S& s, int n) {
  while (n > 0) {
    const int m = n < 8 ? n : 8;
    s.put64(0x3030303030303030ull >> (8 * (8 - m)), (uint32_t)m);
    n -= m;
  }
}

// fmt::format("{}", v) for finite v: the shortest digits that round-trip, fixed notation when the decimal
// exponent lies in [-4, 16), exponent notation otherwise.
template <class S> K2J_HD void put_double(S& s, double v) {
  const DoubleLayout L = double_layout(v);
  if (L.neg) put_char(s, '-');
  if (L.zero) { put_char(s, '0'); return; }
  const int nd = L.nd, e10 = L.e10;
  if (S::kCounting) {
    if (e10 < -4 || e10 >= 16) {
      const int a = e10 < 0 ? -e10 : e10;
      s.skip((uint32_t)(nd + (nd > 1 ? 1 : 0) + 2 + (a < 100 ? 2 : 3)));
    } else if (e10 >= nd - 1) s.skip((uint32_t)(e10 + 1));
    else if (e10 >= 0) s.skip((uint32_t)(nd + 1));
    else s.skip((uint32_t)(nd + 1 - e10));
    return;
  }
  const Digits17 D = digits17(L.dec);
  const int z = 17 - nd;  // leading zeros of the padded string
  if (e10 < -4 || e10 >= 16) {
    s.put64(digits_at(D, z) & 0xffull, 1);
    if (nd > 1) { put_char(s, '.'); put_digits(s, D, z + 1, nd - 1); }
    const int a = e10 < 0 ? -e10 : e10;
    s.put(0x65u | ((e10 < 0 ? 0x2Du : 0x2Bu) << 8), 2);  // 'e' then sign
    if (a < 10) put_char(s, '0');
    put_small(s, (uint32_t)a);
    return;
  }
  if (e10 >= nd - 1) {
    put_digits(s, D, z, nd);
    put_zeros(s, e10 - (nd - 1));
  } else if (e10 >= 0) {
    put_digits(s, D, z, e10 + 1);
    put_char(s, '.');
    put_digits(s, D, z + e10 + 1, nd - e10 - 1);
  } else {
    s.put64(0x303030302E30ull & (~0ull >> (8 * (7 + e10))), (uint32_t)(1 - e10));  // "0." and -e10 - 1 zeros
    put_digits(s, D, z, nd);
  }
}
// TypedMetadataJson.h:172-178: finite values bare, non-finite values quoted.
template <class S> K2J_HD void put_double_value(S& s, double v) {
  if (double_is_finite(v)) { put_double(s, v); return; }
  put_char(s, '"'); put_nonfinite(s, v); put_char(s, '"');
}

// ------------------------------------------------------------------------------------------------
// x87 80-bit emulation of the reference's TSC -> unix-ns converter
//   static_cast<time_t>(static_cast<double>(t - t0_approx) * scale_factor) + t0
// (libkineto/src/ApproximateClock.cpp:83-90), scale_factor being a long double with a 64-bit
// significand `mant` and value mant * 2^(exp-63).  The double-by-extended product is rounded to 64
// significant bits (nearest-even, the x87 default), then truncated toward zero.
// ------------------------------------------------------------------------------------------------
K2J_HD int64_t tsc_to_ns(uint64_t t, uint64_t t0_approx, int64_t t0, uint64_t mant, int exp) {
  if (!(t > t0_approx)) return 0;
  uint64_t diff = t - t0_approx;
  // (double)diff : round to nearest even to 53 bits
  int lz = clz64(diff);
  uint64_t m = diff << lz;         // normalised, top bit set
  int e2 = 63 - lz;                // diff = m * 2^(e2-63)
  uint64_t m53 = m >> 11, rem = m & 0x7FF;
  if (rem > 0x400 || (rem == 0x400 && (m53 & 1))) m53++;
  if (m53 >> 53) { m53 >>= 1; e2++; }
  // m53 has 53 bits: value = m53 * 2^(e2-52)
  // product = m53 * mant * 2^(e2-52 + exp-63); 53+64 = up to 117 bits
  uint64_t plo = m53 * mant, phi = umulhi64(m53, mant);
  // normalise the 128-bit product to 64 significant bits with round-to-nearest-even
  int plz = phi ? clz64(phi) : 64 + clz64(plo);
  int bitlen = 128 - plz;  // >= 64 here because mant has its top bit set and m53 >= 2^52
  int drop = bitlen - 64;
  uint64_t sig;
  if (drop <= 0) { sig = plo; drop = 0; }
  else {
    sig = (phi << (64 - drop)) | (plo >> drop);  // drop in 1..63
    uint64_t lost = plo & ((1ull << drop) - 1), half = 1ull << (drop - 1);
    if (lost > half || (lost == half && (sig & 1))) { sig++; if (sig == 0) { sig = 1ull << 63; drop++; } }
  }
  // value = sig * 2^(drop + e2 - 52 + exp - 63)
  int sh = drop + e2 - 52 + exp - 63;
  int64_t r;
  // sig has its top bit set, so any non-negative shift is >= 2^63: the x87 store yields the
  // "integer indefinite" value 0x8000000000000000.
  if (sh >= 0) r = (int64_t)0x8000000000000000ull;
  else r = (-sh) < 64 ? (int64_t)(sig >> (-sh)) : 0;
  return (int64_t)((uint64_t)r + (uint64_t)t0);
}

}  // namespace k2j
