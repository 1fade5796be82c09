// Linear-attention mixers with a matrix state per head: the token-by-token recurrence, the short
// causal convolution that may come before it, and the per-head norm and gate that come after it.
//
// State of head h of a request: S [dk, dv] in float32, kept as [dv, dk] (a column's dk entries are
// contiguous) in the request's slot. With a decay d_t [dk] per token (one factor per key channel):
//
//   decay rule:  S <- diag(d_t) S + k_t v_t^T;                         o_t = S^T q_t
//   delta rule:  S <- diag(d_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//
// The columns of S never meet: column j of S and element j of v, u and o make a recurrence of their
// own. So a CTA takes (request, head, a run of columns), a column is held by L threads of a warp
// (16 key channels each, in registers), and the sums over key channels go through that lane group in a
// fixed order. Tokens are taken in chunks: the CTA stages the chunk's q, k, v (and beta) and works out
// the decays in float32, all threads at once, then walks the chunk token by token. A request's result
// is the same bit for bit however its tokens are cut into steps and whatever else the step holds: the
// state is carried in float32 and nothing in a token's arithmetic depends on the chunking.
//
// The decay is d = exp(-c_h * softplus(sign * (z + bias))) with z the output of a projection:
// sign = -1, c_h = 1/tau gives sigmoid(z + bias)^(1/tau); sign = +1, c_h = exp(A_h) gives
// exp(-exp(A_h) softplus(z + bias)).
#include "common.cuh"

namespace ms {

constexpr int SCAN_KPT = 16;      // key channels per thread
constexpr int SCAN_THREADS = 256;

__device__ __forceinline__ float softplusf(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

template <typename TIn, typename TZ, bool DELTA>
__global__ void __launch_bounds__(SCAN_THREADS)
decay_scan_kernel(float* __restrict__ o_out,   // [T, H, dv]
                  float* __restrict__ state,   // [slots, H, dv, dk]
                  const TIn* __restrict__ q, int ld_q, const TIn* __restrict__ k, int ld_k, int qk_group,
                  const TIn* __restrict__ v, int ld_v,
                  const TZ* __restrict__ z, int ld_z, const float* __restrict__ z_bias, const float* __restrict__ decay_coef,
                  float z_sign, const TZ* __restrict__ beta, int ld_beta,
                  const int* __restrict__ cu_q, const int* __restrict__ q_start, const int* __restrict__ state_slot,
                  int H, int dk, int dv, int L, int chunk, float q_scale) {
  extern __shared__ float smem[];
  pdl_prologue();
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int cols = SCAN_THREADS / L;
  const int col = tid / L, l = tid - col * L;
  const int j = blockIdx.z * cols + col;
  const bool active = j < dv;
  const int dkp = L * (SCAN_KPT + 1);  // a lane's 16 channels, then one word of padding: lanes fall on different banks
  float* qs = smem;
  float* ks = qs + (size_t)chunk * dkp;
  float* ds = ks + (size_t)chunk * dkp;
  float* vs = ds + (size_t)chunk * dkp;   // [chunk, cols]
  float* bs = vs + (size_t)chunk * cols;  // [chunk]
  for (int i = tid; i < 3 * chunk * dkp; i += SCAN_THREADS) smem[i] = 0.f;  // channels beyond dk stay zero

  const int t0 = cu_q[r], t1 = cu_q[r + 1];
  const int slot = state_slot[r];
  const bool fresh = q_start[r] == 0;
  float* srow = state + (((size_t)slot * H + h) * dv + (active ? j : 0)) * dk;
  float S[SCAN_KPT];
#pragma unroll
  for (int e = 0; e < SCAN_KPT; ++e) {
    const int i = l * SCAN_KPT + e;
    S[e] = (!fresh && active && i < dk) ? srow[i] : 0.f;
  }
  const int qk_head = h / qk_group;
  const float coef = decay_coef[h];
  __syncthreads();

  for (int c0 = t0; c0 < t1; c0 += chunk) {
    const int n = min(chunk, t1 - c0);
    for (int idx = tid; idx < n * dk; idx += SCAN_THREADS) {
      const int tt = idx / dk, i = idx - tt * dk;
      const size_t tok = (size_t)(c0 + tt);
      const int at = tt * dkp + i + i / SCAN_KPT;
      qs[at] = Elem<TIn>::load(q + tok * ld_q + (size_t)qk_head * dk + i) * q_scale;
      ks[at] = Elem<TIn>::load(k + tok * ld_k + (size_t)qk_head * dk + i);
      const float zz = Elem<TZ>::load(z + tok * ld_z + (size_t)h * dk + i) + z_bias[(size_t)h * dk + i];
      ds[at] = expf(-coef * softplusf(z_sign * zz));
    }
    for (int idx = tid; idx < n * cols; idx += SCAN_THREADS) {
      const int tt = idx / cols, c = idx - tt * cols;
      const int jj = blockIdx.z * cols + c;
      vs[idx] = jj < dv ? Elem<TIn>::load(v + (size_t)(c0 + tt) * ld_v + (size_t)h * dv + jj) : 0.f;
    }
    if (DELTA) {
      for (int tt = tid; tt < n; tt += SCAN_THREADS)
        bs[tt] = 1.0f / (1.0f + expf(-Elem<TZ>::load(beta + (size_t)(c0 + tt) * ld_beta + h)));
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float* qt = qs + tt * dkp + l * (SCAN_KPT + 1);
      const float* kt = ks + tt * dkp + l * (SCAN_KPT + 1);
      const float* dt = ds + tt * dkp + l * (SCAN_KPT + 1);
      const float vj = vs[tt * cols + col];
      // sums over a thread's channels in four interleaved chains (a fixed order), so that the token's
      // critical path is four products deep and not sixteen
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
      if (DELTA) {
        float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int e = 0; e < SCAN_KPT; ++e) {
          S[e] *= dt[e];
          d4[e & 3] = fmaf(kt[e], S[e], d4[e & 3]);
        }
        float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
        for (int off = L >> 1; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float u = bs[tt] * (vj - dot);
#pragma unroll
        for (int e = 0; e < SCAN_KPT; ++e) {
          S[e] = fmaf(kt[e], u, S[e]);
          a4[e & 3] = fmaf(qt[e], S[e], a4[e & 3]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < SCAN_KPT; ++e) {
          S[e] = fmaf(dt[e], S[e], kt[e] * vj);
          a4[e & 3] = fmaf(qt[e], S[e], a4[e & 3]);
        }
      }
      float acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
      for (int off = L >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (l == 0 && active) o_out[((size_t)(c0 + tt) * H + h) * dv + j] = acc;
    }
    __syncthreads();
  }
  if (active) {
#pragma unroll
    for (int e = 0; e < SCAN_KPT; ++e) {
      const int i = l * SCAN_KPT + e;
      if (i < dk) srow[i] = S[e];
    }
  }
}

// Short causal convolution over time per channel, then SiLU, then (for the first `unit_heads` heads of
// `dk` channels) division by the head's Euclidean length: y / sqrt(sum y^2 + unit_eps). The heads after
// those have `dv` channels and are not normalised. Channels are columns [0, C) of the projection's rows;
// w [C, taps], the last tap is the current token's. Inputs before a portion's first token come from the
// request's slot (the last taps - 1 inputs of the portion before), or are zero at the start of a sequence.
// One warp per (token, head).
template <typename T>
__global__ void conv_silu_unit_kernel(float* __restrict__ out, const T* __restrict__ proj, int ld,
                                      const T* __restrict__ conv_state,  // [slots, taps - 1, C]
                                      const float* __restrict__ w, const int* __restrict__ row_of_token,
                                      const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                      const int* __restrict__ state_slot, int num_tokens, int C, int taps, int unit_heads,
                                      int dk, int other_heads, int dv, float unit_eps) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const int units = unit_heads + other_heads;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * units) return;
  const int t = (int)(item / units), u = (int)(item - (long long)t * units);
  const bool unit = u < unit_heads;
  const int base = unit ? u * dk : unit_heads * dk + (u - unit_heads) * dv;
  const int size = unit ? dk : dv;
  const int row = row_of_token[t];
  const int local = t - cu_q[row];
  const bool started = q_start[row] > 0;
  const T* st = conv_state + (size_t)state_slot[row] * (taps - 1) * C;
  float ss = 0.f;
  for (int c = lane; c < size; c += 32) {
    const int ch = base + c;
    float acc = 0.f;
    for (int jt = 0; jt < taps; ++jt) {
      const int back = taps - 1 - jt;
      const int at = local - back;
      float x = 0.f;
      if (at >= 0) x = Elem<T>::load(proj + (size_t)(t - back) * ld + ch);
      else if (started) x = Elem<T>::load(st + (size_t)(taps - 1 + at) * C + ch);
      acc = fmaf(w[(size_t)ch * taps + jt], x, acc);
    }
    const float y = acc / (1.0f + expf(-acc));
    out[(size_t)t * C + ch] = y;
    ss += y * y;
  }
  if (!unit) return;
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + unit_eps);
  for (int c = lane; c < size; c += 32) out[(size_t)t * C + base + c] *= inv;
}

// The slot's last taps - 1 inputs after this step, oldest first. One thread per (request, channel);
// entry s takes what was entry s + len when the portion is shorter than the history kept.
template <typename T>
__global__ void conv_state_update_kernel(T* __restrict__ conv_state, const T* __restrict__ proj, int ld,
                                         const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                         const int* __restrict__ state_slot, int num_rows, int C, int taps) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)num_rows * C) return;
  const int r = (int)(idx / C), ch = (int)(idx - (long long)r * C);
  const int keep = taps - 1;
  const int t0 = cu_q[r], len = cu_q[r + 1] - t0;
  const bool started = q_start[r] > 0;
  T* st = conv_state + (size_t)state_slot[r] * keep * C + ch;
  for (int s = 0; s < keep; ++s) {
    const int at = len - keep + s;
    float x = 0.f;
    if (at >= 0) x = Elem<T>::load(proj + (size_t)(t0 + at) * ld + ch);
    else if (started) x = Elem<T>::load(st + (size_t)(s + len) * C);
    Elem<T>::store(st + (size_t)s * C, x);
  }
}

// out[t, h * dv + c] = scale * o[t, h, c] / sqrt(mean_c o^2 + eps) * w[c] * act(gate[t, h * dv + c]),
// act = SiLU (0) or sigmoid (1). One warp per (token, head).
template <typename T>
__global__ void head_norm_gate_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ o, const float* __restrict__ w,
                                      const T* __restrict__ gate, int ld_gate, int num_tokens, int H, int dv, float eps,
                                      float scale, int gate_kind) {
  pdl_prologue();
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)num_tokens * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const float* src = o + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += src[c] * src[c];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float g = Elem<T>::load(gate + (size_t)t * ld_gate + (size_t)h * dv + c);
    const float sg = 1.0f / (1.0f + expf(-g));
    const float a = gate_kind == 0 ? g * sg : sg;
    Elem<T>::store(out + (size_t)t * ld_out + (size_t)h * dv + c, scale * ((src[c] * inv) * w[c]) * a);
  }
}

template <typename TIn, typename TZ, bool DELTA>
int launch_scan(float* o_out, float* state, const void* q, int ld_q, const void* k, int ld_k, int qk_group, const void* v, int ld_v,
                const void* z, int ld_z, const float* z_bias, const float* decay_coef, float z_sign, const void* beta, int ld_beta,
                const int* cu_q, const int* q_start, const int* state_slot, int num_rows, int H, int dk, int dv, float q_scale,
                cudaStream_t stream) {
  int L = 1;
  while (L * SCAN_KPT < dk) L <<= 1;
  const int cols = SCAN_THREADS / L;
  const int dkp = L * (SCAN_KPT + 1);
  const int per_token = (3 * dkp + cols + 1) * (int)sizeof(float);
  int chunk = (40 * 1024) / per_token;
  chunk = chunk > 32 ? 32 : (chunk < 1 ? 1 : chunk);
  const size_t smem = (size_t)chunk * per_token;
  auto kernel = decay_scan_kernel<TIn, TZ, DELTA>;
  const dim3 grid(num_rows, H, (dv + cols - 1) / cols);
  MS_LAUNCH(kernel, grid, SCAN_THREADS, smem, stream, o_out, state, (const TIn*)q, ld_q, (const TIn*)k, ld_k, qk_group,
            (const TIn*)v, ld_v, (const TZ*)z, ld_z, z_bias, decay_coef, z_sign, (const TZ*)beta, ld_beta, cu_q, q_start, state_slot,
            H, dk, dv, L, chunk, q_scale);
  return 0;
}

}  // namespace ms

using namespace ms;

// in_dtype: of q, k, v; z_dtype: of z and beta. delta: 0 decay rule, 1 delta rule.
MS_EXPORT int ms_decay_scan(float* o_out, float* state, const void* q, int ld_q, const void* k, int ld_k, int qk_group,
                            const void* v, int ld_v, const void* z, int ld_z, const float* z_bias, const float* decay_coef,
                            float z_sign, const void* beta, int ld_beta, const int* cu_q, const int* q_start,
                            const int* state_slot, int num_rows, int H, int dk, int dv, float q_scale, int delta, int in_dtype,
                            int z_dtype, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  MS_CHECK_ARG(H > 0 && dk > 0 && dv > 0 && dk <= 32 * SCAN_KPT, "decay_scan: key size %d is outside 1..%d", dk, 32 * SCAN_KPT);
  MS_CHECK_ARG(qk_group > 0 && H % qk_group == 0, "decay_scan: %d heads are not a multiple of the group of %d", H, qk_group);
  MS_CHECK_ARG(!delta || beta != nullptr, "decay_scan: the delta rule needs beta");
#define MS_SCAN(TIN, TZZ, D)                                                                                                  \
  return launch_scan<TIN, TZZ, D>(o_out, state, q, ld_q, k, ld_k, qk_group, v, ld_v, z, ld_z, z_bias, decay_coef, z_sign, beta, \
                                  ld_beta, cu_q, q_start, state_slot, num_rows, H, dk, dv, q_scale, stream)
  if (in_dtype == MS_F32 && z_dtype == MS_F32) {
    if (delta) MS_SCAN(float, float, true);
    MS_SCAN(float, float, false);
  }
  if (in_dtype == MS_F32 && z_dtype == MS_BF16) {
    if (delta) MS_SCAN(float, __nv_bfloat16, true);
    MS_SCAN(float, __nv_bfloat16, false);
  }
  if (in_dtype == MS_BF16 && z_dtype == MS_BF16) {
    if (delta) MS_SCAN(__nv_bfloat16, __nv_bfloat16, true);
    MS_SCAN(__nv_bfloat16, __nv_bfloat16, false);
  }
#undef MS_SCAN
  return ms::fail("decay_scan: unsupported dtypes (%d, %d)", in_dtype, z_dtype);
}

MS_EXPORT int ms_conv_silu_unit(float* out, const void* proj, int ld, const void* conv_state, const float* w,
                                const int* row_of_token, const int* cu_q, const int* q_start, const int* state_slot,
                                int num_tokens, int C, int taps, int unit_heads, int dk, int other_heads, int dv, float unit_eps,
                                int dtype, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  MS_CHECK_ARG(taps >= 1 && C == unit_heads * dk + other_heads * dv, "conv_silu_unit: %d channels are not %d x %d + %d x %d", C,
               unit_heads, dk, other_heads, dv);
  const long long items = (long long)num_tokens * (unit_heads + other_heads);
  const int warps = 8;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(conv_silu_unit_kernel<float>, blocks, warps * 32, 0, stream, out, (const float*)proj, ld, (const float*)conv_state, w,
              row_of_token, cu_q, q_start, state_slot, num_tokens, C, taps, unit_heads, dk, other_heads, dv, unit_eps);
  else
    MS_LAUNCH(conv_silu_unit_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, out, (const __nv_bfloat16*)proj, ld,
              (const __nv_bfloat16*)conv_state, w, row_of_token, cu_q, q_start, state_slot, num_tokens, C, taps, unit_heads, dk,
              other_heads, dv, unit_eps);
  return 0;
}

MS_EXPORT int ms_conv_state_update(void* conv_state, const void* proj, int ld, const int* cu_q, const int* q_start,
                                   const int* state_slot, int num_rows, int C, int taps, int dtype, cudaStream_t stream) {
  if (num_rows == 0 || taps <= 1) return 0;
  const long long items = (long long)num_rows * C;
  const unsigned blocks = (unsigned)((items + 255) / 256);
  if (dtype == MS_F32)
    MS_LAUNCH(conv_state_update_kernel<float>, blocks, 256, 0, stream, (float*)conv_state, (const float*)proj, ld, cu_q, q_start,
              state_slot, num_rows, C, taps);
  else
    MS_LAUNCH(conv_state_update_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)conv_state,
              (const __nv_bfloat16*)proj, ld, cu_q, q_start, state_slot, num_rows, C, taps);
  return 0;
}

MS_EXPORT int ms_head_norm_gate(void* out, int ld_out, const float* o, const float* w, const void* gate, int ld_gate,
                                int num_tokens, int H, int dv, float eps, float scale, int gate_kind, int dtype,
                                cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const long long items = (long long)num_tokens * H;
  const int warps = 8;
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
  if (dtype == MS_F32)
    MS_LAUNCH(head_norm_gate_kernel<float>, blocks, warps * 32, 0, stream, (float*)out, ld_out, o, w, (const float*)gate, ld_gate,
              num_tokens, H, dv, eps, scale, gate_kind);
  else
    MS_LAUNCH(head_norm_gate_kernel<__nv_bfloat16>, blocks, warps * 32, 0, stream, (__nv_bfloat16*)out, ld_out, o, w,
              (const __nv_bfloat16*)gate, ld_gate, num_tokens, H, dv, eps, scale, gate_kind);
  return 0;
}
