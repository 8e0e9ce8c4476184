// Generator of tests/golden/cutlass_tables.json: evaluates the reference's literal
// quantisation expressions (MixedGemm src/reorder.cu:164-248) with CUTLASS's own host
// NumericConverter classes - the third-party code the reference delegates its rounding
// to - and prints the resulting tables as JSON.  Run by make_golden.py; needs a CUTLASS
// header tree (not part of this repository).  Nothing at test time depends on CUTLASS:
// only the emitted JSON is committed.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "cutlass/numeric_conversion.h"
#include "cutlass/numeric_types.h"

using fp4_t = cutlass::float_e2m1_t;
using fp6_t = cutlass::float_e3m2_t;
using fp8_t = cutlass::float_e4m3_t;
using sf_t = cutlass::float_ue8m0_t;
using bf16_t = cutlass::bfloat16_t;

static cutlass::NumericConverter<fp4_t, float> cvt4;
static cutlass::NumericConverter<fp6_t, float> cvt6;
static cutlass::NumericConverter<fp8_t, float> cvt8;
static cutlass::NumericConverter<sf_t, float> cvtSF;
static cutlass::NumericConverter<bf16_t, float> cvtBF;

static float bf16_bits_to_float(uint16_t b) {
  uint32_t u = uint32_t(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

static float fclamp(float x, float a, float b) { return std::fmax(a, std::fmin(b, x)); }

static uint8_t encode(float t, int fmt) {
  bf16_t r = cvtBF(t);
  if (fmt == 0) return cvt4(float(r)).storage & 0xF;
  if (fmt == 1) return cvt6(float(r)).storage & 0x3F;
  return cvt8(float(r)).storage;
}

static const float kMax[3] = {6.f, 28.f, 448.f};

// scale byte for a group maximum (src/reorder.cu:179-185)
static uint8_t scale_byte(float maxv, int fmt, float* scale_out) {
  float scale;
  if (maxv == 0) scale = 0.5f;
  else scale = float(cvtBF(ldexpf(1.0f, static_cast<int>(std::ceil(std::log2(maxv / kMax[fmt]))))));
  if (scale_out) *scale_out = scale;
  return cvtSF(scale).storage;
}

static uint32_t lcg(uint32_t& s) { s = s * 1664525u + 1013904223u; return s >> 8; }

int main() {
  std::printf("{\n");
  const char* names[3] = {"e2m1", "e3m2", "e4m3"};
  // 1. magnitude code of every integer the chain can produce
  for (int f = 0; f < 3; ++f) {
    std::printf("\"codes_%s\": [", names[f]);
    for (int n = 0; n <= int(kMax[f]); ++n) std::printf("%s%u", n ? "," : "", encode(float(n), f));
    std::printf("],\n");
    std::printf("\"negzero_%s\": %u,\n", names[f], encode(-0.0f, f));
  }
  // 2. scale byte for every finite bf16 magnitude, as [first_bits, byte] change points
  for (int f = 0; f < 3; ++f) {
    std::printf("\"scale_%s\": [", names[f]);
    int prev = -1;
    bool first = true;
    for (uint32_t a = 0x0080; a < 0x7F80; ++a) {  // normal bf16 magnitudes
      int b = scale_byte(bf16_bits_to_float(uint16_t(a)), f, nullptr);
      if (b != prev) {
        std::printf("%s[%u,%d]", first ? "" : ",", a, b);
        first = false;
        prev = b;
      }
    }
    std::printf("],\n");
    std::printf("\"scale_zero_%s\": %u,\n", names[f], scale_byte(0.f, f, nullptr));
  }
  // 3. whole groups through the full chain: random bf16 patterns in a moderate exponent
  //    range plus adversarial maxima (MAX*2^k and its bf16 neighbours, zeros, -0)
  std::printf("\"groups\": [\n");
  uint32_t seed = 12345u;
  bool firstg = true;
  for (int f = 0; f < 3; ++f) {
    for (int g = 0; g < 48; ++g) {
      uint16_t bits[32];
      for (int i = 0; i < 32; ++i) {
        uint32_t r = lcg(seed);
        uint32_t e = 110 + (r % 30);  // exponents 2^-17 .. 2^12
        bits[i] = uint16_t(((r >> 5) & 0x8000) | (e << 7) | ((r >> 8) & 0x7F));
      }
      if (g % 8 == 1) {  // exact MAX * 2^k maximum
        float m = kMax[f] * ldexpf(1.f, (g % 5) - 2);
        uint32_t u; std::memcpy(&u, &m, 4);
        for (int i = 0; i < 32; ++i) bits[i] = uint16_t((bits[i] & 0x8000) | ((bits[i] & 0x7FFF) % ((u >> 16) + 1)));
        bits[g % 32] = uint16_t(u >> 16);
      } else if (g % 8 == 2 || g % 8 == 3) {  // one bf16 ulp above / below MAX * 2^k
        float m = kMax[f] * ldexpf(1.f, (g % 7) - 3);
        uint32_t u; std::memcpy(&u, &m, 4);
        uint16_t top = uint16_t((u >> 16) + (g % 8 == 2 ? 1 : -1));
        for (int i = 0; i < 32; ++i) bits[i] = uint16_t((bits[i] & 0x8000) | ((bits[i] & 0x7FFF) % (top + 1)));
        bits[(g * 7) % 32] = uint16_t(top | 0x8000);
      } else if (g % 8 == 4) {  // all zero with a few negative zeros
        for (int i = 0; i < 32; ++i) bits[i] = (i % 5 == 0) ? 0x8000 : 0x0000;
      } else if (g % 8 == 5) {  // ties: halves and integers
        for (int i = 0; i < 32; ++i) {
          float v = 0.5f * float(int(lcg(seed) % 25)) * ((lcg(seed) & 1) ? -1.f : 1.f);
          uint32_t u; std::memcpy(&u, &v, 4);
          bits[i] = uint16_t(u >> 16);
        }
      }
      float maxv = 0;
      for (int i = 0; i < 32; ++i) {
        float a = std::fabs(bf16_bits_to_float(bits[i]));
        maxv = maxv > a ? maxv : a;
      }
      float scale;
      int sf = scale_byte(maxv, f, &scale);
      float r_scale = 1.0 / scale;
      std::printf("%s{\"fmt\":%d,\"bits\":[", firstg ? "" : ",\n", f);
      firstg = false;
      for (int i = 0; i < 32; ++i) std::printf("%s%u", i ? "," : "", bits[i]);
      std::printf("],\"sf\":%d,\"codes\":[", sf);
      for (int i = 0; i < 32; ++i) {
        float t = fclamp(std::round(bf16_bits_to_float(bits[i]) * r_scale), -kMax[f], kMax[f]);
        std::printf("%s%u", i ? "," : "", encode(t, f));
      }
      std::printf("]}");
    }
  }
  std::printf("\n]\n}\n");
  return 0;
}
