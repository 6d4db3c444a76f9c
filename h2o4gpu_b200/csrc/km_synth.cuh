// Counter-based synthetic data on the device (benchmark inputs that do not fit
// host memory).  Philox4x32-10 keyed by the seed; the counter is (global row,
// column group, stream), so any shard of the matrix can be produced on any GPU
// and shards never overlap.  Distributions follow the benchmark configurations:
// Gaussian mixtures (component per row from a weight table) and the image-like
// sparse integer matrix.
#pragma once

#include "km_common.cuh"

namespace km {

struct Philox {
  static __device__ __forceinline__ uint4 run(uint4 c, uint2 key) {
    const unsigned int M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      unsigned int hi0 = __umulhi(M0, c.x), lo0 = M0 * c.x;
      unsigned int hi1 = __umulhi(M1, c.z), lo1 = M1 * c.z;
      c = make_uint4(hi1 ^ c.y ^ key.x, lo1, hi0 ^ c.w ^ key.y, lo0);
      key.x += 0x9E3779B9u;
      key.y += 0xBB67AE85u;
    }
    return c;
  }
};

__device__ __forceinline__ float u01(unsigned int b) { return ((b >> 8) + 0.5f) * (1.0f / 16777216.0f); }

// cdf: n_comp cumulative weights (last = 1).  centers: n_comp x d row-major.
template <typename T>
__global__ void __launch_bounds__(256)
synth_kernel(T* __restrict__ X, size_t rows, int d, size_t row0, int kind,
             const T* __restrict__ centers, int n_comp, const float* __restrict__ cdf, T sigma,
             unsigned long long seed) {
  const uint2 key = make_uint2((unsigned int)seed, (unsigned int)(seed >> 32));
  const int groups = (d + 3) / 4;
  const size_t total = rows * (size_t)groups;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    size_t r = i / groups;
    int gcol = (int)(i - r * groups);
    size_t gr = row0 + r;
    uint4 rnd = Philox::run(make_uint4((unsigned int)gr, (unsigned int)(gr >> 32), (unsigned int)gcol, 0u), key);
    T v[4];
    if (kind == 1) {
      unsigned int b[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        bool zero = (b[e] >> 8) < 13421773u;  // 0.8 * 2^24
        v[e] = zero ? (T)0 : (T)(1 + ((b[e] & 0xffu) * 255u >> 8));
      }
    } else {
      // component of this row: one draw on stream 1
      uint4 rc = Philox::run(make_uint4((unsigned int)gr, (unsigned int)(gr >> 32), 0u, 1u), key);
      float u = u01(rc.x);
      int lo = 0, hi = n_comp - 1;
      while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (cdf[mid] < u) lo = mid + 1; else hi = mid;
      }
      float r1 = sqrtf(-2.0f * logf(u01(rnd.x)));
      float r2 = sqrtf(-2.0f * logf(u01(rnd.z)));
      float s1, c1, s2, c2;
      sincospif(2.0f * u01(rnd.y), &s1, &c1);
      sincospif(2.0f * u01(rnd.w), &s2, &c2);
      float g[4] = {r1 * c1, r1 * s1, r2 * c2, r2 * s2};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int col = gcol * 4 + e;
        T base = (col < d) ? centers[(size_t)lo * d + col] : (T)0;
        v[e] = base + sigma * (T)g[e];
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int col = gcol * 4 + e;
      if (col < d) X[r * (size_t)d + col] = v[e];
    }
  }
}

}  // namespace km
