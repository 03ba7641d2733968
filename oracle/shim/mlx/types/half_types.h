// TEST INFRASTRUCTURE - stand-in for the one MLX header the reference's CPU
// codec translation units include ("mlx/types/half_types.h"). MLX itself is not
// installed where this oracle is built, so this shim supplies the two names the
// reference uses, with IEEE-754 round-to-nearest-even conversions:
//   mlx::core::float16_t  - the compiler's native _Float16 (RNE by definition)
//   mlx::core::bfloat16_t - a 16-bit storage struct, float -> bf16 by RNE on the
//                           dropped 16 mantissa bits, NaN kept quiet.
// numpy's astype(float16) and torch's .to(bfloat16) round the same way, which
// is how the parity tests cross-check these conversions.
#pragma once

#include <cstdint>
#include <cstring>

namespace mlx {
namespace core {

typedef _Float16 float16_t;

struct bfloat16_t {
  uint16_t bits;

  bfloat16_t() = default;

  bfloat16_t(float f) {
    uint32_t u;
    std::memcpy(&u, &f, sizeof(u));
    if ((u & 0x7fffffffu) > 0x7f800000u) {
      bits = static_cast<uint16_t>((u >> 16) | 0x0040u); // quiet NaN
    } else {
      u += 0x7fffu + ((u >> 16) & 1u); // round to nearest, ties to even
      bits = static_cast<uint16_t>(u >> 16);
    }
  }

  operator float() const {
    uint32_t u = static_cast<uint32_t>(bits) << 16;
    float f;
    std::memcpy(&f, &u, sizeof(f));
    return f;
  }
};

} // namespace core
} // namespace mlx
