// A recurrent mixer's kernels: the short causal convolution in front of it, and the gated delta
// rule with one decay per head and key channel.
//
// State per request (float32, in state slots): the last taps - 1 inputs of the convolution, and
// per head the matrix S [DK key channels, dv value channels].
//
// Per token and head, in this order (all float32):
//   g = exp(-exp(A_log) * softplus(a + dt_bias))       one per key channel
//   S = diag(g) S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q
//   out = o / sqrt(mean(o^2) + eps) * w_norm * sigmoid(gate)
// The recurrence walks a request's tokens of this step one after the other, so a prompt cut
// anywhere, or decoded token by token, runs the same arithmetic in the same order.
#include "common.cuh"

#ifndef DELTA_DK
#define DELTA_DK 64
#endif
#define DELTA_MAX_TAPS 16

__device__ __forceinline__ int request_of(const int* __restrict__ cu_seqlens, int num_seqs, int t) {
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// ---------------------------------------------------------------------------------
// y[t, c] = silu(sum_j taps[c, j] * in[t - (K - 1 - j), c]); inputs before the portion come from
// the request's state (row K - 2 is the latest), zeros for a fresh request. Channels
// [0, unit_channels) are then made unit vectors in runs of `unit_dim` (x / sqrt(sum x^2 + unit_eps)),
// the first `scaled_channels` of them also multiplied by `scale`.
// One block per token; the inputs are columns [col0, col0 + C) of the projected rows.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ proj, int stride, int col0, int C, int K,
                                  const float* __restrict__ taps, const float* __restrict__ state,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                  int num_seqs, int unit_channels, int unit_dim, float unit_eps,
                                  int scaled_channels, float scale, float* __restrict__ y) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float val[];  // [C]
  const int t = blockIdx.x;
  const int seq = request_of(cu_seqlens, num_seqs, t);
  const int start = cu_seqlens[seq];
  const float* tail = state + (size_t)state_slots[seq] * (K - 1) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int back = K - 1 - j;  // how many tokens before t
      const int src = t - back;
      float x;
      if (src >= start) x = to_f32(proj[(size_t)src * stride + col0 + c]);
      else x = tail[(size_t)(K - 1 - (start - src)) * C + c];
      acc += taps[(size_t)c * K + j] * x;
    }
    val[c] = acc / (1.f + expf(-acc));
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int head = warp; head * unit_dim < unit_channels; head += nwarps) {
    float ss = 0.f;
    for (int i = lane; i < unit_dim; i += 32) ss += val[head * unit_dim + i] * val[head * unit_dim + i];
    ss = warp_sum(ss);
    const float r = rsqrtf(ss + unit_eps) * (head * unit_dim < scaled_channels ? scale : 1.f);
    for (int i = lane; i < unit_dim; i += 32) val[head * unit_dim + i] *= r;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) y[(size_t)t * C + c] = val[c];
}

extern "C" int omnia_short_conv(const void* proj, int stride, int col0, int channels, int taps_count,
                                const float* taps, const float* state, const int* cu_seqlens,
                                const int* state_slots, int num_seqs, int unit_channels, int unit_dim,
                                float unit_eps, int scaled_channels, float scale, float* y, int tokens,
                                int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (taps_count < 1 || taps_count > DELTA_MAX_TAPS || (unit_channels && unit_dim < 1)) return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (size_t)channels;
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(short_conv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    launch_pdl(short_conv_kernel<T>, tokens, 256, smem, stream, (const T*)proj, stride, col0, channels, taps_count,
               taps, state, cu_seqlens, state_slots, num_seqs, unit_channels, unit_dim, unit_eps, scaled_channels,
               scale, y);
  });
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// The recurrence. Grid (heads, requests); a block has P threads for each of the head's dv value
// channels: thread (j, p) keeps rows p, p + P, ... of column j of S in registers. The block of
// head 0 also moves the request's convolution state on (nothing else reads it in this kernel).
//
// conv:  float32 [tokens, C]: q heads (G x DK) | k heads (G x DK) | v heads (H x dv), after the
//        convolution, SiLU and (q, k) the unit norm.
// rows:  the projected rows [tokens, stride] of element type T; columns: raw convolution inputs at
//        in_col (C wide), beta's logit at beta_col (H), the decay's logits at a_col (H x DK) and the
//        output gate's logits at gate_col (H x dv). a and gate may live in other tensors (own strides).
template <typename T, int P, int MAX_THREADS>
__global__ void __launch_bounds__(MAX_THREADS) delta_rule_kernel(const float* __restrict__ conv, int C, int G, int H, int dv,
                                  const T* __restrict__ rows, int stride, int in_col, int beta_col,
                                  const T* __restrict__ a_rows, int a_stride, const T* __restrict__ gate_rows,
                                  int gate_stride, const float* __restrict__ A_log,
                                  const float* __restrict__ dt_bias, const float* __restrict__ norm_w, float eps,
                                  float* __restrict__ S_state, float* __restrict__ conv_state, int K,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                  T* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DK = DELTA_DK;
  constexpr int R = (DK + P - 1) / P;
  __shared__ float ks[DK], qs[DK], gs[DK];
  __shared__ float beta_s;
  __shared__ float scratch[33];
  const int head = blockIdx.x, seq = blockIdx.y;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  const int slot = state_slots[seq];
  const int j = threadIdx.x / P, p = threadIdx.x % P;
  const bool live = j < dv;
  const int group = head / (H / G);
  const float rate = expf(A_log[head]);

  float S[R];
  float* mine = S_state + (((size_t)slot * H + head) * DK) * dv + j;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = p + P * i;
    S[i] = (live && r < DK) ? mine[(size_t)r * dv] : 0.f;
  }
  const float nw = live ? norm_w[j] : 0.f;

  for (int t = begin; t < end; ++t) {
    __syncthreads();
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      qs[i] = conv[(size_t)t * C + group * DK + i];
      ks[i] = conv[(size_t)t * C + (G + group) * DK + i];
      const float z = to_f32(a_rows[(size_t)t * a_stride + head * DK + i]) + dt_bias[head * DK + i];
      const float softplus = z > 20.f ? z : log1pf(expf(z));
      gs[i] = expf(-rate * softplus);
    }
    if (threadIdx.x == 0) beta_s = 1.f / (1.f + expf(-to_f32(rows[(size_t)t * stride + beta_col + head])));
    __syncthreads();
    const float v = live ? conv[(size_t)t * C + 2 * G * DK + head * dv + j] : 0.f;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = p + P * i;
      if (r < DK) {
        S[i] *= gs[r];
        dot += S[i] * ks[r];
      }
    }
#pragma unroll
    for (int o = 1; o < P; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float u = beta_s * (v - dot);
    float o_j = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = p + P * i;
      if (r < DK) {
        S[i] += ks[r] * u;
        o_j += S[i] * qs[r];
      }
    }
#pragma unroll
    for (int o = 1; o < P; o <<= 1) o_j += __shfl_xor_sync(0xffffffffu, o_j, o);
    const float ss = block_sum((live && p == 0) ? o_j * o_j : 0.f, scratch);
    if (live && p == 0) {
      const float gate = to_f32(gate_rows[(size_t)t * gate_stride + head * dv + j]);
      const float y = o_j * rsqrtf(ss / (float)dv + eps) * nw / (1.f + expf(-gate));
      out[(size_t)t * H * dv + head * dv + j] = from_f32<T>(y);
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = p + P * i;
    if (live && r < DK) mine[(size_t)r * dv] = S[i];
  }

  if (head == 0 && K > 1 && end > begin) {
    // The convolution's state after this portion: its last K - 1 inputs, the older ones still
    // from the state before when the portion is shorter than that.
    float* tail = conv_state + (size_t)slot * (K - 1) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float keep[DELTA_MAX_TAPS];
      for (int row = 0; row < K - 1; ++row) {
        const int src = end - (K - 1 - row);  // row K - 2 is the latest token
        keep[row] = src >= begin ? to_f32(rows[(size_t)src * stride + in_col + c])
                                 : tail[(size_t)(row + (end - begin)) * C + c];
      }
      for (int row = 0; row < K - 1; ++row) tail[(size_t)row * C + c] = keep[row];
    }
  }
}

extern "C" int omnia_delta_dk(void) { return DELTA_DK; }

extern "C" int omnia_delta_rule(const float* conv, int C, int G, int H, int dv, const void* rows, int stride,
                                int in_col, int beta_col, const void* a_rows, int a_stride, const void* gate_rows,
                                int gate_stride, const float* A_log, const float* dt_bias, const float* norm_w,
                                float eps, float* S_state, float* conv_state, int taps_count, const int* cu_seqlens,
                                const int* state_slots, int num_seqs, void* out, int dtype, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (G < 1 || H % G != 0 || dv < 1 || dv > 1024 || taps_count < 1 || taps_count > DELTA_MAX_TAPS ||
      C != 2 * G * DELTA_DK + H * dv)
    return (int)cudaErrorInvalidValue;
  const dim3 grid(H, num_seqs);
#define OMNIA_DELTA_LAUNCH(P, MAX_THREADS)                                                                        \
  launch_pdl(delta_rule_kernel<T, P, MAX_THREADS>, grid, dim3((dv * P + 31) / 32 * 32), 0, stream, conv, C, G, H, dv, \
             (const T*)rows, stride, in_col, beta_col, (const T*)a_rows, a_stride, (const T*)gate_rows, gate_stride, \
             A_log, dt_bias, norm_w, eps, S_state, conv_state, taps_count, cu_seqlens, state_slots, (T*)out)
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (dv * 4 <= 512) OMNIA_DELTA_LAUNCH(4, 512);
    else if (dv * 4 <= 1024) OMNIA_DELTA_LAUNCH(4, 1024);
    else if (dv * 2 <= 1024) OMNIA_DELTA_LAUNCH(2, 1024);
    else OMNIA_DELTA_LAUNCH(1, 1024);
  });
#undef OMNIA_DELTA_LAUNCH
  return OMNIA_LAUNCH_RESULT();
}
