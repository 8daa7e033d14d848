// A 64 x 64 output tile on the CUDA cores with IEEE float32 multiply-adds, for products whose
// operands are reached through index arithmetic of the caller's (rows gathered by an index,
// one weight matrix per head or per expert): the caller gives two functors, a(m, k) and
// b(k, n), that return one element as float32 (zero outside the operand), and gets the
// accumulators of a 4 x 4 piece per thread.  256 threads; thread t holds rows
// (t / 16) * 4 + i and columns (t % 16) * 4 + j of the tile.
#pragma once
#include "common.cuh"

namespace rl {

constexpr int TG_M = 64, TG_N = 64, TG_K = 16;

struct TileGemmSmem {
  float a[TG_K][TG_M + 1];
  float b[TG_K][TG_N + 1];
};

template <class LoadA, class LoadB>
__device__ __forceinline__ void tile_gemm(float (&acc)[4][4], int k_total, LoadA load_a, LoadB load_b,
                                          TileGemmSmem& s) {
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int k0 = 0; k0 < k_total; k0 += TG_K) {
#pragma unroll
    for (int i = tid; i < TG_K * TG_M; i += 256) {
      const int kk = i & (TG_K - 1), m = i >> 4;
      s.a[kk][m] = load_a(m, k0 + kk);
    }
#pragma unroll
    for (int i = tid; i < TG_K * TG_N; i += 256) {
      const int kk = i & (TG_K - 1), n = i >> 4;
      s.b[kk][n] = load_b(k0 + kk, n);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TG_K; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = s.a[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = s.b[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
}

// The same with two weight operands that share a: two sets of accumulators (a gate and an up
// projection of one input).
template <class LoadA, class LoadB, class LoadC>
__device__ __forceinline__ void tile_gemm_pair(float (&acc_b)[4][4], float (&acc_c)[4][4], int k_total, LoadA load_a,
                                               LoadB load_b, LoadC load_c, TileGemmSmem& s, float (&c_s)[TG_K][TG_N + 1]) {
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  for (int k0 = 0; k0 < k_total; k0 += TG_K) {
#pragma unroll
    for (int i = tid; i < TG_K * TG_M; i += 256) {
      const int kk = i & (TG_K - 1), m = i >> 4;
      s.a[kk][m] = load_a(m, k0 + kk);
    }
#pragma unroll
    for (int i = tid; i < TG_K * TG_N; i += 256) {
      const int kk = i & (TG_K - 1), n = i >> 4;
      s.b[kk][n] = load_b(k0 + kk, n);
      c_s[kk][n] = load_c(k0 + kk, n);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TG_K; ++kk) {
      float av[4], bv[4], cv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = s.a[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        bv[j] = s.b[kk][tx * 4 + j];
        cv[j] = c_s[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc_b[i][j] = fmaf(av[i], bv[j], acc_b[i][j]);
          acc_c[i][j] = fmaf(av[i], cv[j], acc_c[i][j]);
        }
    }
    __syncthreads();
  }
}

}  // namespace rl
