// Host-side pixel helpers: finite check over raw bf16/fp32 bit patterns and bf16 CHW -> RGB8 HWC
// conversion.  Compiled with -fno-fast-math -ffp-contract=off so that scale, offset and the
// x255 step are three individually rounded fp32 operations, exactly as the device kernel
// (pointwise.cu: rgb8_kernel) computes them; the two are compared bit-for-bit in the tests.
// Behavioural counterpart of the reference's only native file,
// deploy/solar_wm/shared/media/pixels.c:7-34.
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace {

template <typename Word, Word ExpMask>
bool all_finite(const Word* words, std::size_t count) {
  Word seen = 0;
  for (std::size_t i = 0; i < count; ++i) seen |= static_cast<Word>((words[i] & ExpMask) == ExpMask);
  return seen == 0;
}

inline float bf16_bits_to_float(std::uint16_t bits) {
  const std::uint32_t wide = static_cast<std::uint32_t>(bits) << 16;
  float value;
  std::memcpy(&value, &wide, sizeof(value));
  return value;
}

}  // namespace

// 1 if every element is finite, 0 if any Inf/NaN, -1 for an unsupported width.
extern "C" int solar_host_all_finite(const void* data, std::size_t count, int bits) {
  if (bits == 16) return all_finite<std::uint16_t, 0x7f80u>(static_cast<const std::uint16_t*>(data), count);
  if (bits == 32) return all_finite<std::uint32_t, 0x7f800000u>(static_cast<const std::uint32_t*>(data), count);
  return -1;
}

// Returns 1 on success, 0 if a NaN pixel was met (output then unspecified past that pixel).
extern "C" int solar_host_rgb8_bf16(const std::uint16_t* chw, std::size_t height, std::size_t width,
                                    std::size_t stride_c, std::size_t stride_y, std::size_t stride_x,
                                    const float* mean3, const float* std3, std::uint8_t* hwc) {
  for (std::size_t y = 0; y < height; ++y) {
    for (std::size_t x = 0; x < width; ++x) {
      std::uint8_t* px = hwc + (y * width + x) * 3;
      for (std::size_t c = 0; c < 3; ++c) {
        float v = bf16_bits_to_float(chw[c * stride_c + y * stride_y + x * stride_x]);
        v = v * std3[c];
        v = v + mean3[c];
        if (std::isnan(v)) return 0;
        if (v < 0.0f) v = 0.0f;
        else if (v > 1.0f) v = 1.0f;
        v = v * 255.0f;
        px[c] = static_cast<std::uint8_t>(std::nearbyintf(v));
      }
    }
  }
  return 1;
}
