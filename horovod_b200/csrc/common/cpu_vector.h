// Vectorised CPU kernels for the 16-bit float formats on the host data path:
// element-wise sum and scale, and the Adasum building blocks (dot product /
// squared norms, scaled add). Each function picks an AVX2 + F16C
// implementation at run time when the CPU has both and otherwise runs the
// scalar software conversion; both give the same results bit for bit
// (conversions round to nearest even in either case).
//
// Parity: horovod/common/half.cc:28-76 (cpuid check, F16C fp16 sum),
// horovod/common/ops/collective_operations.h:91-127 (AVX scale),
// horovod/common/ops/adasum/adasum.h:438-557 (AVX fp16 dot/norm/scaled add);
// bfloat16 is new here.
#pragma once

#include <cstdint>

namespace hvd {

// True when the AVX2 + F16C paths are in use on this machine.
bool CpuHasF16C();
// Forces the scalar paths (tests compare them with the vector paths).
void CpuVectorForceScalar(bool on);

void HalfSum(uint16_t* dst, const uint16_t* src, int64_t n);   // dst += src (fp16)
void BF16Sum(uint16_t* dst, const uint16_t* src, int64_t n);   // dst += src (bf16)
void HalfScale(uint16_t* buf, int64_t n, float factor);        // buf *= factor
void BF16Scale(uint16_t* buf, int64_t n, float factor);
// dot = sum a*b, na = sum a*a, nb = sum b*b, accumulated in double.
void HalfDotNorms(const uint16_t* a, const uint16_t* b, int64_t n, double* dot, double* na,
                  double* nb);
void BF16DotNorms(const uint16_t* a, const uint16_t* b, int64_t n, double* dot, double* na,
                  double* nb);
// out = ca * a + cb * b, computed in double and rounded once to fp32 and once
// to the 16-bit type (out may alias a or b).
void HalfScaledAdd(uint16_t* out, const uint16_t* a, const uint16_t* b, int64_t n, double ca,
                   double cb);
void BF16ScaledAdd(uint16_t* out, const uint16_t* a, const uint16_t* b, int64_t n, double ca,
                   double cb);

}  // namespace hvd
