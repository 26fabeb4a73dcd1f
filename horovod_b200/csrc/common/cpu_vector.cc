#include "cpu_vector.h"

#include <atomic>

#include "half.h"

#if defined(__x86_64__)
#include <immintrin.h>
#define HVD_X86 1
#define HVD_AVX2 __attribute__((target("avx2,f16c,fma")))
#else
#define HVD_X86 0
#endif

namespace hvd {

namespace {

std::atomic<bool> g_force_scalar{false};

bool Detect() {
#if HVD_X86
  return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c") &&
         __builtin_cpu_supports("fma");
#else
  return false;
#endif
}

bool UseVector() {
  static const bool has = Detect();
  return has && !g_force_scalar.load(std::memory_order_relaxed);
}

#if HVD_X86
// ---- fp16 <-> fp32, 8 lanes ------------------------------------------------
HVD_AVX2 inline __m256 LoadHalf8(const uint16_t* p) {
  return _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(p)));
}
HVD_AVX2 inline void StoreHalf8(uint16_t* p, __m256 v) {
  _mm_storeu_si128(reinterpret_cast<__m128i*>(p),
                   _mm256_cvtps_ph(v, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
}
// ---- bf16 <-> fp32, 8 lanes --------------------------------------------------
HVD_AVX2 inline __m256 LoadBF8(const uint16_t* p) {
  const __m128i raw = _mm_loadu_si128(reinterpret_cast<const __m128i*>(p));
  return _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(raw), 16));
}
HVD_AVX2 inline void StoreBF8(uint16_t* p, __m256 v) {
  // Round to nearest even on the 16 dropped bits; NaN keeps its sign and
  // exponent and gets a quiet mantissa bit (what FloatToBF16Bits does).
  const __m256i x = _mm256_castps_si256(v);
  const __m256i lsb = _mm256_and_si256(_mm256_srli_epi32(x, 16), _mm256_set1_epi32(1));
  const __m256i rounded =
      _mm256_srli_epi32(_mm256_add_epi32(x, _mm256_add_epi32(_mm256_set1_epi32(0x7fff), lsb)), 16);
  const __m256i quiet =
      _mm256_or_si256(_mm256_srli_epi32(x, 16), _mm256_set1_epi32(0x40));
  const __m256i is_nan = _mm256_castps_si256(_mm256_cmp_ps(v, v, _CMP_UNORD_Q));
  const __m256i r = _mm256_blendv_epi8(rounded, quiet, is_nan);
  // 32 -> 16 bits without saturation: the values fit 16 bits already.
  const __m256i packed = _mm256_packus_epi32(_mm256_and_si256(r, _mm256_set1_epi32(0xffff)),
                                             _mm256_setzero_si256());
  const __m256i ordered = _mm256_permute4x64_epi64(packed, 0xd8);
  _mm_storeu_si128(reinterpret_cast<__m128i*>(p), _mm256_castsi256_si128(ordered));
}

HVD_AVX2 void HalfSumV(uint16_t* d, const uint16_t* s, int64_t n) {
  for (int64_t i = 0; i + 8 <= n; i += 8) StoreHalf8(d + i, _mm256_add_ps(LoadHalf8(d + i), LoadHalf8(s + i)));
}
HVD_AVX2 void BF16SumV(uint16_t* d, const uint16_t* s, int64_t n) {
  for (int64_t i = 0; i + 8 <= n; i += 8) StoreBF8(d + i, _mm256_add_ps(LoadBF8(d + i), LoadBF8(s + i)));
}
HVD_AVX2 void HalfScaleV(uint16_t* p, int64_t n, float f) {
  const __m256 vf = _mm256_set1_ps(f);
  for (int64_t i = 0; i + 8 <= n; i += 8) StoreHalf8(p + i, _mm256_mul_ps(LoadHalf8(p + i), vf));
}
HVD_AVX2 void BF16ScaleV(uint16_t* p, int64_t n, float f) {
  const __m256 vf = _mm256_set1_ps(f);
  for (int64_t i = 0; i + 8 <= n; i += 8) StoreBF8(p + i, _mm256_mul_ps(LoadBF8(p + i), vf));
}

// Adds the products of 8 float pairs to two double accumulators (4 lanes each).
HVD_AVX2 inline void AccumulateProducts(__m256 x, __m256 y, __m256d* lo, __m256d* hi) {
  *lo = _mm256_fmadd_pd(_mm256_cvtps_pd(_mm256_castps256_ps128(x)),
                        _mm256_cvtps_pd(_mm256_castps256_ps128(y)), *lo);
  *hi = _mm256_fmadd_pd(_mm256_cvtps_pd(_mm256_extractf128_ps(x, 1)),
                        _mm256_cvtps_pd(_mm256_extractf128_ps(y, 1)), *hi);
}
HVD_AVX2 inline double Sum4(__m256d v) {
  alignas(32) double t[4];
  _mm256_store_pd(t, v);
  return (t[0] + t[1]) + (t[2] + t[3]);
}

template <bool HALF>
HVD_AVX2 int64_t DotNormsV(const uint16_t* a, const uint16_t* b, int64_t n, double* dot,
                           double* na, double* nb) {
  __m256d d0 = _mm256_setzero_pd(), d1 = d0, a0 = d0, a1 = d0, b0 = d0, b1 = d0;
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 x = HALF ? LoadHalf8(a + i) : LoadBF8(a + i);
    const __m256 y = HALF ? LoadHalf8(b + i) : LoadBF8(b + i);
    AccumulateProducts(x, y, &d0, &d1);
    AccumulateProducts(x, x, &a0, &a1);
    AccumulateProducts(y, y, &b0, &b1);
  }
  *dot += Sum4(_mm256_add_pd(d0, d1));
  *na += Sum4(_mm256_add_pd(a0, a1));
  *nb += Sum4(_mm256_add_pd(b0, b1));
  return i;
}

template <bool HALF>
HVD_AVX2 int64_t ScaledAddV(uint16_t* out, const uint16_t* a, const uint16_t* b, int64_t n,
                            double ca, double cb) {
  const __m256d vca = _mm256_set1_pd(ca), vcb = _mm256_set1_pd(cb);
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 x = HALF ? LoadHalf8(a + i) : LoadBF8(a + i);
    const __m256 y = HALF ? LoadHalf8(b + i) : LoadBF8(b + i);
    // ca * x + cb * y in double, rounded to float once (as the scalar path does).
    const __m256d lo = _mm256_add_pd(
        _mm256_mul_pd(vca, _mm256_cvtps_pd(_mm256_castps256_ps128(x))),
        _mm256_mul_pd(vcb, _mm256_cvtps_pd(_mm256_castps256_ps128(y))));
    const __m256d hi = _mm256_add_pd(
        _mm256_mul_pd(vca, _mm256_cvtps_pd(_mm256_extractf128_ps(x, 1))),
        _mm256_mul_pd(vcb, _mm256_cvtps_pd(_mm256_extractf128_ps(y, 1))));
    const __m256 r = _mm256_set_m128(_mm256_cvtpd_ps(hi), _mm256_cvtpd_ps(lo));
    if (HALF)
      StoreHalf8(out + i, r);
    else
      StoreBF8(out + i, r);
  }
  return i;
}
#endif  // HVD_X86

}  // namespace

bool CpuHasF16C() { return UseVector(); }
void CpuVectorForceScalar(bool on) { g_force_scalar.store(on); }

void HalfSum(uint16_t* d, const uint16_t* s, int64_t n) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) {
    HalfSumV(d, s, n);
    i = n & ~int64_t(7);
  }
#endif
  for (; i < n; ++i) d[i] = FloatToHalfBits(HalfBitsToFloat(d[i]) + HalfBitsToFloat(s[i]));
}

void BF16Sum(uint16_t* d, const uint16_t* s, int64_t n) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) {
    BF16SumV(d, s, n);
    i = n & ~int64_t(7);
  }
#endif
  for (; i < n; ++i) d[i] = FloatToBF16Bits(BF16BitsToFloat(d[i]) + BF16BitsToFloat(s[i]));
}

void HalfScale(uint16_t* p, int64_t n, float f) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) {
    HalfScaleV(p, n, f);
    i = n & ~int64_t(7);
  }
#endif
  for (; i < n; ++i) p[i] = FloatToHalfBits(HalfBitsToFloat(p[i]) * f);
}

void BF16Scale(uint16_t* p, int64_t n, float f) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) {
    BF16ScaleV(p, n, f);
    i = n & ~int64_t(7);
  }
#endif
  for (; i < n; ++i) p[i] = FloatToBF16Bits(BF16BitsToFloat(p[i]) * f);
}

void HalfDotNorms(const uint16_t* a, const uint16_t* b, int64_t n, double* dot, double* na,
                  double* nb) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) i = DotNormsV<true>(a, b, n, dot, na, nb);
#endif
  for (; i < n; ++i) {
    const double x = HalfBitsToFloat(a[i]), y = HalfBitsToFloat(b[i]);
    *dot += x * y;
    *na += x * x;
    *nb += y * y;
  }
}

void BF16DotNorms(const uint16_t* a, const uint16_t* b, int64_t n, double* dot, double* na,
                  double* nb) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) i = DotNormsV<false>(a, b, n, dot, na, nb);
#endif
  for (; i < n; ++i) {
    const double x = BF16BitsToFloat(a[i]), y = BF16BitsToFloat(b[i]);
    *dot += x * y;
    *na += x * x;
    *nb += y * y;
  }
}

void HalfScaledAdd(uint16_t* out, const uint16_t* a, const uint16_t* b, int64_t n, double ca,
                   double cb) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) i = ScaledAddV<true>(out, a, b, n, ca, cb);
#endif
  for (; i < n; ++i)
    out[i] = FloatToHalfBits(static_cast<float>(ca * HalfBitsToFloat(a[i]) +
                                                cb * HalfBitsToFloat(b[i])));
}

void BF16ScaledAdd(uint16_t* out, const uint16_t* a, const uint16_t* b, int64_t n, double ca,
                   double cb) {
  int64_t i = 0;
#if HVD_X86
  if (UseVector()) i = ScaledAddV<false>(out, a, b, n, ca, cb);
#endif
  for (; i < n; ++i)
    out[i] = FloatToBF16Bits(static_cast<float>(ca * BF16BitsToFloat(a[i]) +
                                                cb * BF16BitsToFloat(b[i])));
}

}  // namespace hvd
