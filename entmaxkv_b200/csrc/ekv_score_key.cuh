// Order-preserving integer keys of stored page scores (top-k selection).
#pragma once

#include "ekv_common.cuh"

namespace ekv {

// Monotone unsigned key of a stored score: larger score <=> larger key.
template <typename T> struct ScoreKey;
template <> struct ScoreKey<__half> {
  using Key = uint32_t;
  static constexpr int BITS = 16;
  static __device__ __forceinline__ Key of_bits(uint32_t u) { return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u); }
  static __device__ __forceinline__ Key of(const __half* p, int i) {
    return of_bits(reinterpret_cast<const unsigned short*>(p)[i]);
  }
  static __device__ __forceinline__ Key of_value(__half v) { return of_bits(__half_as_ushort(v)); }
};
template <> struct ScoreKey<__nv_bfloat16> {
  using Key = uint32_t;
  static constexpr int BITS = 16;
  static __device__ __forceinline__ Key of_bits(uint32_t u) { return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u); }
  static __device__ __forceinline__ Key of(const __nv_bfloat16* p, int i) {
    return of_bits(reinterpret_cast<const unsigned short*>(p)[i]);
  }
  static __device__ __forceinline__ Key of_value(__nv_bfloat16 v) { return of_bits(__bfloat16_as_ushort(v)); }
};
template <> struct ScoreKey<float> {
  using Key = uint32_t;
  static constexpr int BITS = 32;
  static __device__ __forceinline__ Key of_bits(uint32_t u) { return (u & 0x80000000u) ? ~u : (u | 0x80000000u); }
  static __device__ __forceinline__ Key of(const float* p, int i) { return of_bits(__float_as_uint(p[i])); }
  static __device__ __forceinline__ Key of_value(float v) { return of_bits(__float_as_uint(v)); }
};

}  // namespace ekv
