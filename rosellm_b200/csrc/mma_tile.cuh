// A 64 x 64 output tile of a bfloat16 product on the tensor cores (mma.sync m16n8k16, float32
// accumulation), for products whose operand rows are reached through index arithmetic of the
// caller's (rows gathered by an index, one weight matrix per head or per expert).  Both
// operands have their inner index contiguous: the caller gives row_a(m) and row_b(n), the
// address of element 0 of row m of A and of row n of B (nullptr: a row of zeros).  128 threads;
// warp w holds rows (w / 2) * 32 .. + 32 and columns (w % 2) * 32 .. + 32 as 2 x 4 pieces of
// 16 x 8; lane (g = lane / 4, t = lane % 4) holds of piece (mi, ni) the elements
// (g, 2t), (g, 2t + 1), (g + 8, 2t), (g + 8, 2t + 1).
// VEC: every row address is 16-byte aligned and the inner size a multiple of 8 (16-byte loads);
// otherwise elements are fetched one by one.
#pragma once
#include "common.cuh"

namespace rl {

constexpr int MT_M = 64, MT_N = 64, MT_K = 32, MT_LD = MT_K + 8;

// Three stages: the next two K blocks of both operands are on their way (cp.async) while this
// one is used.
constexpr int MT_STAGES = 3;
struct MmaTileSmem {
  __nv_bfloat16 a[MT_STAGES][MT_M][MT_LD];
  __nv_bfloat16 b[MT_STAGES][MT_N][MT_LD];
};

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"((uint32_t)__cvta_generic_to_shared(row)));
}

// 64 rows x MT_K elements of an operand into shared memory, zeros beyond k_total and for null rows.
// VEC: by cp.async (the caller commits and waits); otherwise through registers, element by element.
template <bool VEC, class Row>
__device__ __forceinline__ void mma_stage(__nv_bfloat16 (*dst)[MT_LD], Row row, int k0, int k_total) {
  for (int i = threadIdx.x; i < 64 * (MT_K / 8); i += 128) {
    const int m = i / (MT_K / 8), kv = (i % (MT_K / 8)) * 8;
    const __nv_bfloat16* src = row(m);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (src != nullptr && k0 + kv < k_total) {
      if (VEC) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(&dst[m][kv])),
                     "l"(src + k0 + kv)
                     : "memory");
        continue;
      } else {
        __nv_bfloat16 e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] = k0 + kv + j < k_total ? src[k0 + kv + j] : __float2bfloat16_rn(0.f);
        v = *reinterpret_cast<const uint4*>(e);
      }
    }
    *reinterpret_cast<uint4*>(&dst[m][kv]) = v;
  }
}

__device__ __forceinline__ void mma_step(float (&acc)[2][4][4], const __nv_bfloat16 (*a_s)[MT_LD],
                                         const __nv_bfloat16 (*b_s)[MT_LD]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int m0 = (warp >> 1) * 32, n0 = (warp & 1) * 32;
#pragma unroll
  for (int kk = 0; kk < MT_K; kk += 16) {
    uint32_t af[2][4], bf[4][2];
    // four 8 x 8 pieces an instruction: A as (rows, k), (rows + 8, k), (rows, k + 8), (rows + 8, k + 8);
    // B (stored [n][k]) as (n, k), (n, k + 8), (n + 8, k), (n + 8, k + 8)
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
      const __nv_bfloat16* pa = &a_s[m0 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk + (lane >> 4) * 8];
      ldmatrix_x4(af[mi][0], af[mi][1], af[mi][2], af[mi][3], pa);
    }
#pragma unroll
    for (int ni = 0; ni < 4; ni += 2) {
      const __nv_bfloat16* pb = &b_s[n0 + ni * 8 + (lane & 7) + (lane >> 4) * 8][kk + ((lane >> 3) & 1) * 8];
      ldmatrix_x4(bf[ni][0], bf[ni][1], bf[ni + 1][0], bf[ni + 1][1], pb);
    }
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) mma_bf16_16x8x16(acc[mi][ni], af[mi], bf[ni]);
  }
}

__device__ __forceinline__ void mma_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void mma_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One commit group a K block, also where a block does not exist (an empty group): so "all but
// the newest MT_STAGES - 1 groups are complete" always means "this iteration's block has landed".
template <bool VEC, class RowA, class RowB>
__device__ __forceinline__ void mma_tile(float (&acc)[2][4][4], int k_total, RowA row_a, RowB row_b,
                                         MmaTileSmem& s) {
#pragma unroll
  for (int st = 0; st < MT_STAGES - 1; ++st) {
    if (st * MT_K < k_total) {
      mma_stage<VEC>(s.a[st], row_a, st * MT_K, k_total);
      mma_stage<VEC>(s.b[st], row_b, st * MT_K, k_total);
    }
    mma_commit();
  }
  int buf = 0, fill = MT_STAGES - 1;
  for (int k0 = 0; k0 < k_total; k0 += MT_K) {
    const int ahead = k0 + (MT_STAGES - 1) * MT_K;
    if (ahead < k_total) {  // into the stage that the iteration before has finished with
      mma_stage<VEC>(s.a[fill], row_a, ahead, k_total);
      mma_stage<VEC>(s.b[fill], row_b, ahead, k_total);
    }
    mma_commit();
    mma_wait<MT_STAGES - 1>();
    __syncthreads();
    mma_step(acc, s.a[buf], s.b[buf]);
    __syncthreads();  // the stage may be written again
    buf = buf + 1 == MT_STAGES ? 0 : buf + 1;
    fill = fill + 1 == MT_STAGES ? 0 : fill + 1;
  }
}

// Two weight operands that share A (a gate and an up projection of one input).
template <bool VEC, class RowA, class RowB, class RowC>
__device__ __forceinline__ void mma_tile_pair(float (&acc_b)[2][4][4], float (&acc_c)[2][4][4], int k_total,
                                              RowA row_a, RowB row_b, RowC row_c, MmaTileSmem& s,
                                              __nv_bfloat16 (*c_s)[MT_N][MT_LD]) {
#pragma unroll
  for (int st = 0; st < MT_STAGES - 1; ++st) {
    if (st * MT_K < k_total) {
      mma_stage<VEC>(s.a[st], row_a, st * MT_K, k_total);
      mma_stage<VEC>(s.b[st], row_b, st * MT_K, k_total);
      mma_stage<VEC>(c_s[st], row_c, st * MT_K, k_total);
    }
    mma_commit();
  }
  int buf = 0, fill = MT_STAGES - 1;
  for (int k0 = 0; k0 < k_total; k0 += MT_K) {
    const int ahead = k0 + (MT_STAGES - 1) * MT_K;
    if (ahead < k_total) {
      mma_stage<VEC>(s.a[fill], row_a, ahead, k_total);
      mma_stage<VEC>(s.b[fill], row_b, ahead, k_total);
      mma_stage<VEC>(c_s[fill], row_c, ahead, k_total);
    }
    mma_commit();
    mma_wait<MT_STAGES - 1>();
    __syncthreads();
    mma_step(acc_b, s.a[buf], s.b[buf]);
    mma_step(acc_c, s.a[buf], c_s[buf]);
    __syncthreads();
    buf = buf + 1 == MT_STAGES ? 0 : buf + 1;
    fill = fill + 1 == MT_STAGES ? 0 : fill + 1;
  }
}

// f(row, column, value) for every element of the tile this thread holds.
template <class F>
__device__ __forceinline__ void mma_for_each(const float (&acc)[2][4][4], F f) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int m0 = (warp >> 1) * 32, n0 = (warp & 1) * 32;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        f(m0 + mi * 16 + g + (c >= 2 ? 8 : 0), n0 + ni * 8 + 2 * t + (c & 1), mi, ni, c);
}

}  // namespace rl
