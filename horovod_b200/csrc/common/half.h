// Software conversions between fp32 and the two 16-bit float formats, for the
// CPU data path (the GPU kernels use hardware conversions).
//
// Parity: horovod/common/half.h:44-140 (fp16 only there; bf16 is new here).
#pragma once

#include <cstdint>
#include <cstring>

namespace hvd {

inline float HalfBitsToFloat(uint16_t h) {
  uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      // subnormal: renormalise
      int shift = 0;
      while ((man & 0x400u) == 0) {
        man <<= 1;
        ++shift;
      }
      man &= 0x3ffu;
      bits = sign | ((127 - 15 - shift + 1) << 23) | (man << 13);
    }
  } else if (exp == 0x1f) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + (127 - 15)) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t FloatToHalfBits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t abs = x & 0x7fffffffu;
  if (abs >= 0x7f800000u) {  // inf / nan
    return static_cast<uint16_t>(sign | 0x7c00u |
                                 ((abs > 0x7f800000u) ? 0x200u : 0));
  }
  if (abs >= 0x477ff000u) {  // rounds to >= 65520 -> inf
    return static_cast<uint16_t>(sign | 0x7c00u);
  }
  if (abs < 0x38800000u) {  // result is subnormal or zero
    if (abs < 0x33000000u) return static_cast<uint16_t>(sign);
    int exp = static_cast<int>(abs >> 23);
    uint32_t man = (abs & 0x7fffffu) | 0x800000u;
    int shift = 126 - exp;  // 14..24
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1u))) ++half_man;
    return static_cast<uint16_t>(sign | half_man);
  }
  // normal: round to nearest even on the 13 dropped bits
  uint32_t r = abs + 0xfffu + ((abs >> 13) & 1u);
  return static_cast<uint16_t>(sign | ((r - 0x38000000u) >> 13));
}

inline float BF16BitsToFloat(uint16_t b) {
  uint32_t bits = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t FloatToBF16Bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((x >> 16) | 0x40u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7fffu + lsb;
  return static_cast<uint16_t>(x >> 16);
}

}  // namespace hvd
