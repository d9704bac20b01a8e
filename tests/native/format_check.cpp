// CPU harness around kineto_b200/csrc/k2j_format.cuh: exports batch formatters so the Python tests
// can compare the product's integer / timestamp / double / TSC routines with independent answers.
#include <cstdint>
#include <cstring>
#include <string>
#include "k2j_format.cuh"

extern "C" {
// Each result is written NUL-terminated at out + i*stride.
void fc_doubles(const double* v, int64_t n, char* out, int stride) {
  for (int64_t i = 0; i < n; i++) {
    k2j::StringSink s; k2j::put_double_value(s, v[i]);
    k2j::CountSink c; k2j::put_double_value(c, v[i]);
    if (c.n != s.s.size()) s.s = "COUNT_MISMATCH";
    strncpy(out + i * stride, s.s.c_str(), stride);
  }
}
void fc_u64(const uint64_t* v, int64_t n, char* out, int stride) {
  for (int64_t i = 0; i < n; i++) {
    k2j::StringSink s; k2j::put_u64(s, v[i]);
    k2j::CountSink c; k2j::put_u64(c, v[i]);
    if (c.n != s.s.size()) s.s = "COUNT_MISMATCH";
    strncpy(out + i * stride, s.s.c_str(), stride);
  }
}
void fc_i64(const int64_t* v, int64_t n, char* out, int stride) {
  for (int64_t i = 0; i < n; i++) {
    k2j::StringSink s; k2j::put_i64(s, v[i]);
    k2j::CountSink c; k2j::put_i64(c, v[i]);
    if (c.n != s.s.size()) s.s = "COUNT_MISMATCH";
    strncpy(out + i * stride, s.s.c_str(), stride);
  }
}
void fc_ts(const int64_t* v, int64_t n, char* out, int stride) {
  for (int64_t i = 0; i < n; i++) {
    k2j::StringSink s; k2j::put_ts(s, v[i]);
    k2j::CountSink c; k2j::put_ts(c, v[i]);
    if (c.n != s.s.size()) s.s = "COUNT_MISMATCH";
    strncpy(out + i * stride, s.s.c_str(), stride);
  }
}
// Product's integer emulation of the converter.
void fc_tsc(const uint64_t* t, int64_t n, uint64_t t0a, int64_t t0, uint64_t mant, int exp, int64_t* out) {
  for (int64_t i = 0; i < n; i++) out[i] = k2j::tsc_to_ns(t[i], t0a, t0, mant, exp);
}
// The same expression the reference evaluates, on this machine's long double (x87 on x86-64).
void fc_tsc_native(const uint64_t* t, int64_t n, uint64_t t0a, int64_t t0, uint64_t mant, int exp, int64_t* out) {
  long double scale_factor = __builtin_ldexpl((long double)mant, exp - 63);
  for (int64_t i = 0; i < n; i++) {
    uint64_t t_approx = t[i];
    out[i] = t_approx > t0a ? static_cast<int64_t>(static_cast<double>(t_approx - t0a) * scale_factor) + t0 : 0;
  }
}
int fc_long_double_mant_dig() { return __LDBL_MANT_DIG__; }
}
