// Mixers with a matrix-valued state per request and head: S_t = diag(w_t) S_(t-1) [- (a_t * u_t)(u_t^T S_(t-1))]
// + k_t v_t^T, o_t = S_t^T r_t, the state [dk, dv] in float32, carried from step to step in a state slot.
//
// Two forms share the kernel (`recurrence_kernel<MODE, ...>`):
//   MODE 0, the generalized delta rule: per key channel a decay w = exp(-decay_scale * sigmoid(w0 + W2 tanh(p)))
//     (p: a low-rank projection of the layer's input), a removal rate a = sigmoid(a' + a_bias), the unit key
//     u = k / sqrt(sum k^2 + unit_eps); the removal term and the decay both read the old state.  Output: each
//     head's o divided by its root mean square, times a weight per (head, column), times sigmoid(g).
//   MODE 1, a gated linear recurrence in which the forget gate also decides what is written: f = l + (1 - l) *
//     sigmoid(f' + f_bias), w = f, k = 1 - f, r = silu(q'), no removal.  Output: each head's o RMS-normed with
//     a weight per column that the heads share.
//
// The inputs are columns of one float32 matrix (the packed projections of the layer's input).  A block owns one
// (request, head): thread j keeps column j of the state in registers, so a token costs no exchange between
// threads.  Tokens are taken in chunks: the block first turns the chunk's projections into the vectors of the
// recurrence (all of it in float32: sigmoids, exponentials, the unit key, the low-rank product), a warp a token,
// into shared memory; then every thread walks the chunk's tokens reading those vectors as broadcasts; then, a
// warp a token again, the chunk's outputs are normalised, gated and written in the activation type.
#include "common.cuh"

namespace rl {

constexpr int REC_CHUNK = 16;  // tokens a chunk

struct RecurParams {
  const float* proj;  // [tokens, ldp]
  long ldp;
  int off_r, off_k, off_v, off_a, off_g, off_w;  // first column of each projection (-1: the form has none)
  const float* a_bias;      // [heads * dk]: the removal rate's bias (0), the forget gate's bias (1)
  const float* w0;          // [heads * dk]: the decay's bias (0), the forget gate's lower bound (1)
  const float* w2;          // [heads * dk, rank] (0)
  int rank;
  const float* out_weight;  // [heads * dv] (0), [dv] (1)
  float* state;             // [slots, heads, dk, dv]
  void* out;                // [tokens, ldo]
  long ldo;
  const int* q_start;
  const int* slots;
  int n_heads, dk, dv;
  float eps, decay_scale, unit_eps;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

template <int MODE, int DKMAX, typename TOut>
__global__ __launch_bounds__(256) void recurrence_kernel(const RecurParams p) {
  extern __shared__ __align__(16) float rec_s[];
  pdl_begin();
  const int req = blockIdx.x, head = blockIdx.y;
  const int slot = p.slots[req];
  if (slot < 0) return;  // a padding row of a captured step
  const int t0 = p.q_start[req], t1 = p.q_start[req + 1];
  const int dk = p.dk, dv = p.dv, j = threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int dvp = (dv + 3) & ~3, rankp = p.rank > 0 ? p.rank : 1;
  // shared memory: W, K, R (, U, AU) [chunk][DKMAX]; V, O [chunk][dvp]; the low-rank input [chunk][rank]
  constexpr int NVEC = MODE == 0 ? 5 : 3;
  float* Ws = rec_s;
  float* Ks = Ws + REC_CHUNK * DKMAX;
  float* Rs = Ks + REC_CHUNK * DKMAX;
  float* Us = Rs + REC_CHUNK * DKMAX;                 // MODE 0 only
  float* AUs = Us + REC_CHUNK * DKMAX;                // MODE 0 only
  float* Vs = rec_s + NVEC * REC_CHUNK * DKMAX;
  float* Os = Vs + REC_CHUNK * dvp;
  float* Ls = Os + REC_CHUNK * dvp;
  float S[DKMAX];
  float* st = p.state + (((size_t)slot * p.n_heads + head) * dk) * dv;
#pragma unroll
  for (int i = 0; i < DKMAX; ++i) S[i] = (i < dk && j < dv) ? st[(size_t)i * dv + j] : 0.f;
  const int c0 = head * dk;  // the head's first key channel
  for (int tc = t0; tc < t1; tc += REC_CHUNK) {
    const int nt = min(REC_CHUNK, t1 - tc);
    __syncthreads();  // the chunk before has been read
    for (int t = warp; t < nt; t += n_warps) {
      const float* row = p.proj + (size_t)(tc + t) * p.ldp;
      if (MODE == 0) {
        for (int r = lane; r < p.rank; r += 32) Ls[t * rankp + r] = tanhf(row[p.off_w + r]);
        __syncwarp();
        float ss = 0.f;
        for (int i = lane; i < DKMAX; i += 32) {
          float w = 0.f, k = 0.f, r = 0.f, a = 0.f;
          if (i < dk) {
            const int c = c0 + i;
            k = row[p.off_k + c];
            r = row[p.off_r + c];
            float wl = p.w0[c];
            const float* w2 = p.w2 + (size_t)c * p.rank;
            for (int q = 0; q < p.rank; ++q) wl = fmaf(w2[q], Ls[t * rankp + q], wl);
            w = expf(-p.decay_scale * sigmoidf_(wl));
            a = sigmoidf_(row[p.off_a + c] + p.a_bias[c]);
          }
          Ws[t * DKMAX + i] = w;
          Ks[t * DKMAX + i] = k;
          Rs[t * DKMAX + i] = r;
          AUs[t * DKMAX + i] = a;
          ss = fmaf(k, k, ss);
        }
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss + p.unit_eps);
        for (int i = lane; i < DKMAX; i += 32) {
          const float u = Ks[t * DKMAX + i] * inv;
          Us[t * DKMAX + i] = u;
          AUs[t * DKMAX + i] *= u;
        }
      } else {
        for (int i = lane; i < DKMAX; i += 32) {
          float w = 0.f, k = 0.f, r = 0.f;
          if (i < dk) {
            const int c = c0 + i;
            const float l = p.w0[c];
            const float f = l + (1.0f - l) * sigmoidf_(row[p.off_a + c] + p.a_bias[c]);
            const float q = row[p.off_r + c];
            w = f;
            k = 1.0f - f;
            r = q * sigmoidf_(q);
          }
          Ws[t * DKMAX + i] = w;
          Ks[t * DKMAX + i] = k;
          Rs[t * DKMAX + i] = r;
        }
      }
      for (int c = lane; c < dvp; c += 32) Vs[t * dvp + c] = c < dv ? row[p.off_v + head * dv + c] : 0.f;
    }
    __syncthreads();
    if (j < dvp) {
      for (int t = 0; t < nt; ++t) {
        const float4* W4 = reinterpret_cast<const float4*>(Ws + t * DKMAX);
        const float4* K4 = reinterpret_cast<const float4*>(Ks + t * DKMAX);
        const float4* R4 = reinterpret_cast<const float4*>(Rs + t * DKMAX);
        const float vj = Vs[t * dvp + j];
        float pj = 0.f;
        if (MODE == 0) {
          const float4* U4 = reinterpret_cast<const float4*>(Us + t * DKMAX);
#pragma unroll
          for (int i = 0; i < DKMAX / 4; ++i) {
            const float4 u = U4[i];
            pj = fmaf(u.x, S[4 * i], fmaf(u.y, S[4 * i + 1], fmaf(u.z, S[4 * i + 2], fmaf(u.w, S[4 * i + 3], pj))));
          }
        }
        float o = 0.f;
        const float4* AU4 = reinterpret_cast<const float4*>(AUs + t * DKMAX);
#pragma unroll
        for (int i = 0; i < DKMAX / 4; ++i) {
          const float4 w = W4[i], k = K4[i], r = R4[i];
          float4 au = make_float4(0.f, 0.f, 0.f, 0.f);
          if (MODE == 0) au = AU4[i];
          float s0 = fmaf(w.x, S[4 * i], fmaf(-au.x, pj, k.x * vj));
          float s1 = fmaf(w.y, S[4 * i + 1], fmaf(-au.y, pj, k.y * vj));
          float s2 = fmaf(w.z, S[4 * i + 2], fmaf(-au.z, pj, k.z * vj));
          float s3 = fmaf(w.w, S[4 * i + 3], fmaf(-au.w, pj, k.w * vj));
          S[4 * i] = s0;
          S[4 * i + 1] = s1;
          S[4 * i + 2] = s2;
          S[4 * i + 3] = s3;
          o = fmaf(s0, r.x, fmaf(s1, r.y, fmaf(s2, r.z, fmaf(s3, r.w, o))));
        }
        Os[t * dvp + j] = o;
      }
    }
    __syncthreads();
    for (int t = warp; t < nt; t += n_warps) {
      float ss = 0.f;
      for (int c = lane; c < dv; c += 32) ss = fmaf(Os[t * dvp + c], Os[t * dvp + c], ss);
      ss = warp_sum(ss);
      const float rn = 1.0f / sqrtf(ss / (float)dv + p.eps);
      const float* row = p.proj + (size_t)(tc + t) * p.ldp;
      TOut* orow = reinterpret_cast<TOut*>(p.out) + (size_t)(tc + t) * p.ldo + (size_t)head * dv;
      for (int c = lane; c < dv; c += 32) {
        float v = Os[t * dvp + c] * rn;
        if (MODE == 0)
          v = v * p.out_weight[head * dv + c] * sigmoidf_(row[p.off_g + head * dv + c]);
        else
          v = v * p.out_weight[c];
        orow[c] = from_f32<TOut>(v);
      }
    }
  }
  if (j < dv) {
#pragma unroll
    for (int i = 0; i < DKMAX; ++i)
      if (i < dk) st[(size_t)i * dv + j] = S[i];
  }
}

template <int MODE, int DKMAX, typename TOut>
static int launch_recurrence(const RecurParams& p, int n_reqs, cudaStream_t stream) {
  const int dvp = (p.dv + 3) & ~3;
  const int threads = (dvp + 31) / 32 * 32;
  const size_t smem = ((size_t)(MODE == 0 ? 5 : 3) * REC_CHUNK * DKMAX + 2 * REC_CHUNK * dvp +
                       (size_t)REC_CHUNK * (p.rank > 0 ? p.rank : 1)) * sizeof(float);
  auto kernel = recurrence_kernel<MODE, DKMAX, TOut>;
  if (smem > 48 * 1024) {
    static bool raised = false;
    if (!raised) {
      note_launch(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      raised = true;
    }
  }
  launch_pdl(kernel, dim3(n_reqs, p.n_heads), threads, smem, stream, p);
  return 0;
}

template <int MODE, typename TOut>
static int dispatch_recurrence(const RecurParams& p, int n_reqs, cudaStream_t stream) {
  if (p.dk <= 16) return launch_recurrence<MODE, 16, TOut>(p, n_reqs, stream);
  if (p.dk <= 32) return launch_recurrence<MODE, 32, TOut>(p, n_reqs, stream);
  if (p.dk <= 64) return launch_recurrence<MODE, 64, TOut>(p, n_reqs, stream);
  if (p.dk <= 128) return launch_recurrence<MODE, 128, TOut>(p, n_reqs, stream);
  return launch_recurrence<MODE, 256, TOut>(p, n_reqs, stream);
}

}  // namespace rl

// mode 0: generalized delta rule; 1: gated recurrence (see the top of this file).  proj: float32 [tokens, ldp]
// holding the projections at the given column offsets; state: float32 [slots, heads, dk, dv], read and written
// for the step's requests (slot < 0: skipped); out: [tokens, heads * dv] of out_dtype, row stride ldo.
RL_EXPORT int rl_recurrence(int mode, int out_dtype, const float* proj, long ldp, int off_r, int off_k, int off_v,
                            int off_a, int off_g, int off_w, const float* a_bias, const float* w0, const float* w2,
                            int rank, const float* out_weight, float* state, void* out, long ldo, const int* q_start,
                            const int* slots, int n_reqs, int n_heads, int dk, int dv, float eps, float decay_scale,
                            float unit_eps, cudaStream_t stream) {
  if (n_reqs <= 0) return 0;
  if (mode < 0 || mode > 1 || n_heads <= 0 || dk <= 0 || dk > 256 || dv <= 0 || dv > 256 || rank < 0 || rank > 1024)
    return -2;
  if (n_heads > 65535) return -2;
  rl::RecurParams p{proj, ldp, off_r, off_k, off_v, off_a, off_g, off_w, a_bias, w0, w2, rank, out_weight, state, out,
                    ldo, q_start, slots, n_heads, dk, dv, eps, decay_scale, unit_eps};
  if (mode == 0) {
    if (out_dtype == RL_F32) rl::dispatch_recurrence<0, float>(p, n_reqs, stream);
    else rl::dispatch_recurrence<0, __nv_bfloat16>(p, n_reqs, stream);
  } else {
    if (out_dtype == RL_F32) rl::dispatch_recurrence<1, float>(p, n_reqs, stream);
    else rl::dispatch_recurrence<1, __nv_bfloat16>(p, n_reqs, stream);
  }
  RL_CHECK_LAUNCH();
  return 0;
}
