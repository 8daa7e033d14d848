// Elementwise steps of gated feed-forward layers.
//
// `gated_act_kernel`: the packed product [gate | up] of a token becomes f(gate, up) per unit
// (gated_act.cuh).  `token_gate_kernel`: a per-token input of a layer, out = gelu_tanh(s) * e
// with e the layer's part of the token's row in a second embedding table (the row is looked
// up by the token id here, so the part never exists as a tensor of its own).
#include "gated_act.cuh"

namespace rl {

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, long ld, int up_at, T* __restrict__ out, long ldo,
                                 int n_rows, int width, int kind, float alpha, float limit) {
  pdl_begin();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)n_rows * width) return;
  const int r = (int)(i / width), f = (int)(i - (long)r * width);
  const T* row = gu + (size_t)r * ld;
  out[(size_t)r * ldo + f] = from_f32<T>(gated_value(to_f32(row[f]), to_f32(row[up_at + f]), kind, alpha, limit));
}

// out[n, j] = gelu_tanh(s[n, j]) * table[id_n, col0 + j] for j < dim, 0 for dim <= j < out_width.
template <typename T>
__global__ void token_gate_kernel(const T* __restrict__ s, long lds, const int* __restrict__ ids,
                                  const T* __restrict__ table, long ldt, int col0, int dim, T* __restrict__ out,
                                  long ldo, int out_width, int n_tokens, int vocab, const int* __restrict__ feedback,
                                  int n_feedback, int* __restrict__ status) {
  pdl_begin();
  const int n = blockIdx.x;
  if (n >= n_tokens) return;
  int id = ids[n];
  if (id < 0 && feedback != nullptr && -id - 1 < n_feedback) id = feedback[-id - 1];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(status, RL_STATUS_BAD_TOKEN);
  for (int j = threadIdx.x; j < out_width; j += blockDim.x) {
    float v = 0.f;
    if (j < dim && !bad) v = gelu_tanh_f32(to_f32(s[(size_t)n * lds + j])) * to_f32(table[(size_t)id * ldt + col0 + j]);
    out[(size_t)n * ldo + j] = from_f32<T>(v);
  }
}

}  // namespace rl

// gu: [rows, >= up_at + width] (row stride ld): gate at column f, up at column up_at + f.
RL_EXPORT int rl_gated_act(int dtype, const void* gu, long ld, int up_at, void* out, long ldo, int n_rows, int width,
                           int kind, float alpha, float limit, cudaStream_t stream) {
  if (n_rows <= 0 || width <= 0) return 0;
  if (kind < 0 || kind > 3) return -2;
  const long total = (long)n_rows * width;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == RL_F32)
    rl::launch_pdl(rl::gated_act_kernel<float>, blocks, 256, 0, stream, (const float*)gu, ld, up_at, (float*)out, ldo,
                   n_rows, width, kind, alpha, limit);
  else
    rl::launch_pdl(rl::gated_act_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gu, ld, up_at,
                   (__nv_bfloat16*)out, ldo, n_rows, width, kind, alpha, limit);
  RL_CHECK_LAUNCH();
  return 0;
}

RL_EXPORT int rl_token_gate(int dtype, const void* s, long lds, const int* ids, const void* table, long ldt, int col0,
                            int dim, void* out, long ldo, int out_width, int n_tokens, int vocab, const int* feedback,
                            int n_feedback, int* status, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (dim <= 0 || out_width < dim || status == nullptr) return -2;
  if (dtype == RL_F32)
    rl::launch_pdl(rl::token_gate_kernel<float>, n_tokens, 64, 0, stream, (const float*)s, lds, ids,
                   (const float*)table, ldt, col0, dim, (float*)out, ldo, out_width, n_tokens, vocab, feedback,
                   n_feedback, status);
  else
    rl::launch_pdl(rl::token_gate_kernel<__nv_bfloat16>, n_tokens, 64, 0, stream, (const __nv_bfloat16*)s, lds, ids,
                   (const __nv_bfloat16*)table, ldt, col0, dim, (__nv_bfloat16*)out, ldo, out_width, n_tokens, vocab,
                   feedback, n_feedback, status);
  RL_CHECK_LAUNCH();
  return 0;
}
