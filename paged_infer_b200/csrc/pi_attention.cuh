// Device helpers shared by the paged-attention decode kernels.
#pragma once
#include <math.h>
#include <stdint.h>

constexpr uint32_t kAttnSpinLimit = 1u << 21;   // polls of a bulk copy's mbarrier before a kernel gives up

__device__ __forceinline__ uint32_t attn_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The G head scores of a token are reduce-scattered over the LPT lanes that share the token.  Lane (within those
// lanes) that ends up owning head g, and the head a lane owns.
template <int G, int LPT>
__device__ __forceinline__ constexpr int attn_owner_lane(int g) {
  int li = 0, n = G, o = 1;
  while (n > 1 && o < LPT) {
    n >>= 1;
    if (g >= n) {
      li |= o;
      g -= n;
    }
    o <<= 1;
  }
  return li;
}
template <int G, int LPT>
__device__ __forceinline__ int attn_owned_head(int li) {
  int g = 0, n = G, o = 1;
  while (n > 1 && o < LPT) {
    n >>= 1;
    if (li & o) g += n;
    o <<= 1;
  }
  return g;
}
