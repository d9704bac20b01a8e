// The emit pass's output sink (see WindowSink).  Like k2j_format.cuh this header also compiles as plain C++
// (K2J_HD drops the CUDA qualifiers), so the window logic can be exercised on a CPU: there the "shared memory"
// window and the "global memory" output are ordinary host arrays.
#pragma once
#include <stdint.h>

#include "k2j_format.cuh"

namespace k2j {

// (hi:lo << s) >> 32 for s in 0..31: the bytes that a left shift by s pushes out of lo, below hi's shifted bytes
K2J_HD uint32_t funnel_l(uint32_t lo, uint32_t hi, uint32_t s) {
#if defined(__CUDA_ARCH__)
  return __funnelshift_l(lo, hi, s);
#else
  return s ? (hi << s) | (lo >> (32u - s)) : hi;
#endif
}
// one 256-bit store to a 32-byte aligned address
K2J_HD void store32(uint8_t* p, uint64_t a, uint64_t b, uint64_t c, uint64_t d) {
#if defined(__CUDA_ARCH__)
  asm volatile("st.global.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(p), "l"(a), "l"(b), "l"(c), "l"(d) : "memory");
#else
  uint64_t v[4] = {a, b, c, d};
  memcpy(p, v, 32);
#endif
}

// ---- output sink: a per-thread window in shared memory, flushed in 32-byte blocks ----------------------
// Every thread owns a window of kWinBytes in shared memory that mirrors the part of its event being written:
// window byte p stands for global address gbase + p, and gbase is 32-byte aligned, so window and output agree
// modulo 32.  Appending is cheap: text arrives in 32-bit pieces, a funnel shift puts each piece at the byte phase
// of the write position, and plain 32-bit stores put it into the window (the word being filled is kept in a
// register and stored again as it grows).  When the window runs out of room the thread writes its complete
// 32-byte blocks to global memory, each as one 256-bit store (a full DRAM sector, so the L2 never has to fetch
// the rest of one), moves the open block to the front of the window and goes on.
// The windows of a warp are interleaved word by word: word k of lane t sits at [k][t], i.e. in bank t wherever
// the lanes' write positions are, so no window access of a warp ever meets a bank conflict.
// The two 8-byte words an event may share with its neighbours are written without knowing the neighbour's
// bytes: every event begins with "\n  {\n   " and ends with "\n  },", so the neighbour's (at most three) bytes
// inside a shared 4-byte half are known constants, and a half that belongs wholly to the neighbour is not
// touched.  Both owners write a shared half with the same bytes.  The other words of an event's first and last
// (partial) block leave as 8-byte stores.
constexpr uint64_t kEventHead8 = 0x2020200A7B20200Aull;  // "\n  {\n   "  first 8 bytes of every event
constexpr uint64_t kEventTail8 = 0x2C7D20200A000000ull;  // "\n  },"      last 5 bytes of every event, in the top bytes
constexpr uint32_t kMinEventBytes = 16;
constexpr int kWinBytes = 160;
constexpr int kWinWords = kWinBytes / 4;
constexpr int kWinStride = 32;              // words between consecutive words of one window (the lanes of a warp)
constexpr int kWinPadWords = 8 * kWinStride;  // after the last warp's windows: the move of the open block reads a whole block,
                                              // which may reach past the end of a window (into the next warp's rows, or this pad)
constexpr uint32_t kWinSlack = 40;          // room that always stays free after ensure(): 32 bytes of small appends that
                                            // do not ask first, and the word past the end that an append may touch
K2J_HD uint64_t pack64(uint32_t lo, uint32_t hi) { return (uint64_t)lo | ((uint64_t)hi << 32); }

struct WindowSink {
  static constexpr bool kCounting = false;
  uint32_t* win;          // word 0 of this thread's window; word k is win[k * kWinStride]
  uint32_t pos;           // window offset of the next byte
  uint32_t carry;         // the 32-bit word being filled: bytes below pos & 3 are set, the rest is zero
  uint32_t w0;            // offset of the event's first 8-byte word in its first block; that block is open while head != 0
  uint32_t head;          // 1 until the event's first block has left, if the event starts inside it
  uint8_t* gbase;         // global address of window byte 0, 32-byte aligned
  K2J_HD uint32_t& W(uint32_t k) const { return win[k * (uint32_t)kWinStride]; }
  K2J_HD uint64_t W64(uint32_t k) const { return pack64(W(k), W(k + 1u)); }  // the 8 bytes from word k on
  K2J_HD void init(uint8_t* dst, uint32_t, uint32_t* window) {
    const uint32_t phase32 = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 31u), phase = phase32 & 7u, sh = 8u * phase;
    win = window; gbase = dst - phase32; pos = phase32; carry = 0u;
    w0 = phase32 & ~7u; head = phase32 ? 1u : 0u;
    const uint64_t w = ((kEventTail8 >> 1) >> (63u - sh)) | (kEventHead8 << sh);
    if (phase < 4u) *reinterpret_cast<uint64_t*>(gbase + w0) = w;
    else *reinterpret_cast<uint32_t*>(gbase + w0 + 4) = (uint32_t)(w >> 32);
  }
  K2J_HD void block_out(uint32_t b) {
    const uint32_t k = 8u * b;
    const uint32_t x0 = W(k), x1 = W(k + 1), x2 = W(k + 2), x3 = W(k + 3), x4 = W(k + 4), x5 = W(k + 5), x6 = W(k + 6), x7 = W(k + 7);
    store32(gbase + 32u * b, pack64(x0, x1), pack64(x2, x3), pack64(x4, x5), pack64(x6, x7));
  }
  // Writes the complete 32-byte blocks of the window to global memory and moves the open block to the front.
  K2J_HD void flush() {
    W(pos >> 2) = carry;
    const uint32_t nb = pos >> 5;
    uint32_t b = 0;
    if (head != 0u && nb != 0u) {  // the event starts inside its first block: whole words only (init wrote the first one)
      for (uint32_t o = w0 + 8u; o < 32u; o += 8u) *reinterpret_cast<uint64_t*>(gbase + o) = W64(o >> 2);
      b = 1; head = 0u;
    }
#if defined(__CUDA_ARCH__)
#pragma unroll 1
#endif
    for (; b + 2u <= nb; b += 2u) {  // two blocks at a time: sixteen loads in flight before the two stores
      const uint32_t k = 8u * b;
      const uint32_t x0 = W(k), x1 = W(k + 1), x2 = W(k + 2), x3 = W(k + 3), x4 = W(k + 4), x5 = W(k + 5), x6 = W(k + 6), x7 = W(k + 7);
      const uint32_t y0 = W(k + 8), y1 = W(k + 9), y2 = W(k + 10), y3 = W(k + 11), y4 = W(k + 12), y5 = W(k + 13), y6 = W(k + 14), y7 = W(k + 15);
      store32(gbase + 32u * b, pack64(x0, x1), pack64(x2, x3), pack64(x4, x5), pack64(x6, x7));
      store32(gbase + 32u * b + 32u, pack64(y0, y1), pack64(y2, y3), pack64(y4, y5), pack64(y6, y7));
    }
    if (b < nb) block_out(b);
    if (nb != 0u) {
      const uint32_t k = 8u * nb;
      const uint32_t x0 = W(k), x1 = W(k + 1), x2 = W(k + 2), x3 = W(k + 3), x4 = W(k + 4), x5 = W(k + 5), x6 = W(k + 6), x7 = W(k + 7);
      W(0) = x0; W(1) = x1; W(2) = x2; W(3) = x3; W(4) = x4; W(5) = x5; W(6) = x6; W(7) = x7;
      gbase += 32u * nb; pos -= 32u * nb;
    }
  }
  // After this call n more bytes fit, with kWinSlack to spare.  n <= kWinBytes - 32 - kWinSlack.
  // On the GPU the lanes of a warp that are executing together flush together, as soon as one of them needs
  // the room: a flush that only some lanes take costs the warp as much as one that all of them take, and windows
  // of a warp fill at about the same rate.  (A flush that comes early only writes the blocks that are complete.)
  K2J_HD void ensure(uint32_t n) {
#if defined(__CUDA_ARCH__)
    if (__any_sync(__activemask(), pos + n + kWinSlack > (uint32_t)kWinBytes)) flush();
#else
    if (pos + n + kWinSlack > (uint32_t)kWinBytes) flush();
#endif
  }
  // append the low `len` (0..4) bytes of w; bytes above len must be zero
  K2J_HD void put(uint32_t w, int len) {
    const uint32_t ph = pos & 3u, s = ph << 3;
    const uint32_t t = carry | (w << s);
    W(pos >> 2) = t;
    carry = ph + (uint32_t)len >= 4u ? funnel_l(w, 0u, s) : t;  // the funnel shift gives w >> (32 - s), and 0 for s = 0
    pos += (uint32_t)len;
  }
  K2J_HD void put4(uint32_t w) {
    const uint32_t s = (pos & 3u) << 3;
    W(pos >> 2) = carry | (w << s);
    carry = funnel_l(w, 0u, s);
    pos += 4u;
  }
  // append the low `len` (0..8) bytes of w; bytes above len must be zero
  K2J_HD void put64(uint64_t w, uint32_t len) {
    const uint32_t lo = (uint32_t)w, hi = (uint32_t)(w >> 32);
    const uint32_t ph = pos & 3u, s = ph << 3, i = pos >> 2;
    const uint32_t t0 = carry | (lo << s), t1 = funnel_l(lo, hi, s), t2 = funnel_l(hi, 0u, s);
    W(i) = t0; W(i + 1) = t1;
    const uint32_t k = (ph + len) >> 2;  // words completed: 0..2
    carry = k == 0u ? t0 : (k == 1u ? t1 : t2);
    pos += len;
  }
  K2J_HD void put8w(uint64_t w) {  // append 8 bytes
    const uint32_t lo = (uint32_t)w, hi = (uint32_t)(w >> 32);
    const uint32_t s = (pos & 3u) << 3, i = pos >> 2;
    W(i) = carry | (lo << s); W(i + 1) = funnel_l(lo, hi, s);
    carry = funnel_l(hi, 0u, s);
    pos += 8u;
  }
  K2J_HD void skip(uint32_t) {}
  template <int N> K2J_HD void lit(const Lit<N>& l) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = 0; i < N / 4; i++) put4(l.w[i]);
    if (N % 4) put(l.w[N / 4], N % 4);
  }
  // `len` bytes from an 8-byte aligned word array, any length: 64 bytes at a time, asking for room first.  The
  // words of a piece are all loaded before the first one is appended: a load that waits behind the append of
  // the word before it (the compiler cannot move it across the window's stores) pays the memory latency once
  // per word instead of once per piece.
  K2J_HD void words(const uint64_t* w, uint32_t len) {
    uint64_t x[8], y[8];
    {
      const uint32_t touched = ((len < 64u ? len : 64u) + 7u) >> 3;  // words read, the partial last one included
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
      for (uint32_t k = 0; k < 8u; k++) x[k] = k < touched ? w[k] : 0ull;
    }
    while (true) {
      const uint32_t n = len < 64u ? len : 64u;
      {  // the piece after this one is on its way while this one is appended
        const uint32_t left = len - n, touched = ((left < 64u ? left : 64u) + 7u) >> 3;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
        for (uint32_t k = 0; k < 8u; k++) y[k] = k < touched ? w[8 + k] : 0ull;
      }
      ensure(n);
      const uint32_t nw = n >> 3;
      const uint32_t s = (pos & 3u) << 3;
      uint32_t i = pos >> 2, c = carry;
      uint64_t last = x[0];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
      for (uint32_t k = 0; k < 8u; k++) {
        if (k < nw) {
          const uint32_t lo = (uint32_t)x[k], hi = (uint32_t)(x[k] >> 32);
          W(i) = c | (lo << s); W(i + 1) = funnel_l(lo, hi, s);
          c = funnel_l(hi, 0u, s);
          i += 2;
        }
        if (k == nw) last = x[k];
      }
      carry = c; pos += 8u * nw;
      const uint32_t rem = n & 7u;
      if (rem) put64(last & (~0ull >> (8u * (8u - rem))), rem);
      len -= n;
      if (len == 0u) break;
      w += 8;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
      for (uint32_t k = 0; k < 8u; k++) x[k] = y[k];
    }
  }
  // `len` bytes from any address: the bytes up to the next 8-byte boundary, then whole words
  K2J_HD void bytes(const uint8_t* src, uint32_t len) {
    const uint32_t a = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 7u);
    const uint64_t* w = reinterpret_cast<const uint64_t*>(src - a);
    if (a != 0u && len != 0u) {
      const uint32_t n = len < 8u - a ? len : 8u - a;
      put64((w[0] >> (8u * a)) & (~0ull >> (8u * (8u - n))), n);
      len -= n; w += 1;
    }
    if (len) words(w, len);
  }
  // Writes what is left: the complete blocks, the complete words of the open block, then the word holding the
  // event's end.  Returns false if the byte count differs from the size the event was given.
  K2J_HD bool finish(const uint8_t* dst, uint32_t size) {
    flush();
    for (uint32_t o = head != 0u ? w0 + 8u : 0u; o + 8u <= pos; o += 8u)  // the event's very first word was written by init
      *reinterpret_cast<uint64_t*>(gbase + o) = W64(o >> 2);
    const uint32_t e = pos & 7u;
    if (e) {
      const uint64_t lo = (pos & 4u) ? pack64(W((pos >> 2) - 1u), carry) : (uint64_t)carry;
      const uint64_t t = lo | (0x20200Aull << (8u * e));  // the next event begins "\n  "
      if (e > 4u) *reinterpret_cast<uint64_t*>(gbase + (pos & ~7u)) = t;
      else *reinterpret_cast<uint32_t*>(gbase + (pos & ~7u)) = (uint32_t)t;
    }
    return gbase + pos == dst + size;
  }
};

}  // namespace k2j
