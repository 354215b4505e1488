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
// One block per token, everything of a token that needs no other token's result:
//   y[t, c] = silu(sum_j taps[c, j] * in[t - (K - 1 - j), c])  for the C convolved channels (q | k | v);
//   inputs before the portion come from the request's state (row K - 2 is the latest), zeros for a
//   fresh request. Channels [0, unit_channels) are then made unit vectors in runs of `unit_dim`
//   (x / sqrt(sum x^2 + unit_eps)), the first `scaled_channels` of them also multiplied by `scale`.
//   decay[t, i] = exp(-exp(A_log[i / unit_dim]) * softplus(a[t, i] + dt_bias[i]))  for i < gate_channels
//   beta[t, h]  = sigmoid(b[t, h])                                                 for h < beta_heads
// Output row (float32): [ y (C) | decay (gate_channels) | beta (beta_heads) ], `out_stride` floats apart.
// The inputs are columns [col0, col0 + C) of the projected rows, beta's logits columns from beta_col.
template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ proj, int stride, int col0, int C, int K,
                                  const float* __restrict__ taps, const float* __restrict__ state,
                                  const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                                  int num_seqs, int unit_channels, int unit_dim, float unit_eps,
                                  int scaled_channels, float scale, const T* __restrict__ a_rows, int a_stride,
                                  const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                  int gate_channels, int beta_col, int beta_heads, float* __restrict__ y,
                                  int out_stride, int chunk) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float val[];  // [chunk]: this block's channels
  const int t = blockIdx.x;
  // Block y of a token takes channels [y chunk, (y + 1) chunk), chunk a multiple of unit_dim, so a
  // unit-normed run never straddles two blocks; and its share of the decays and betas.
  const int c_lo = blockIdx.y * chunk, c_hi = min(C, c_lo + chunk);
  const int seq = request_of(cu_seqlens, num_seqs, t);
  const int start = cu_seqlens[seq];
  const float* tail = state + (size_t)state_slots[seq] * (K - 1) * C;
  float* row = y + (size_t)t * out_stride;
  const int extras = gate_channels + beta_heads;
  const int per = (extras + gridDim.y - 1) / gridDim.y;
  // The loads of the decays' logits are asked for first; they are used last.
  const int e0 = blockIdx.y * per + threadIdx.x;
  float z_first = 0.f;
  if (threadIdx.x < per && e0 < gate_channels) z_first = to_f32(a_rows[(size_t)t * a_stride + e0]);
  for (int c = c_lo + threadIdx.x; c < c_hi; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int src = t - (K - 1 - j);  // K - 1 - j tokens before t
      const float x = src >= start ? to_f32(proj[(size_t)src * stride + col0 + c])
                                   : tail[(size_t)(K - 1 - (start - src)) * C + c];
      acc += taps[(size_t)c * K + j] * x;
    }
    val[c - c_lo] = acc / (1.f + expf(-acc));
  }
  for (int e = blockIdx.y * per + threadIdx.x; e < min(extras, (int)(blockIdx.y + 1) * per); e += blockDim.x) {
    if (e < gate_channels) {
      const float z = (e == e0 ? z_first : to_f32(a_rows[(size_t)t * a_stride + e])) + dt_bias[e];
      const float softplus = z > 20.f ? z : log1pf(expf(z));
      row[C + e] = expf(-expf(A_log[e / unit_dim]) * softplus);
    } else {
      row[C + e] = 1.f / (1.f + expf(-to_f32(proj[(size_t)t * stride + beta_col + e - gate_channels])));
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int c0 = c_lo + warp * unit_dim; c0 < min(c_hi, unit_channels); c0 += nwarps * unit_dim) {
    float ss = 0.f;
    for (int i = lane; i < unit_dim; i += 32) ss += val[c0 - c_lo + i] * val[c0 - c_lo + i];
    ss = warp_sum(ss);
    const float r = rsqrtf(ss + unit_eps) * (c0 < scaled_channels ? scale : 1.f);
    for (int i = lane; i < unit_dim; i += 32) val[c0 - c_lo + i] *= r;
  }
  __syncthreads();
  for (int c = c_lo + threadIdx.x; c < c_hi; c += blockDim.x) row[c] = val[c - c_lo];
}

extern "C" int omnia_short_conv(const void* proj, int stride, int col0, int channels, int taps_count,
                                const float* taps, const float* state, const int* cu_seqlens,
                                const int* state_slots, int num_seqs, int unit_channels, int unit_dim,
                                float unit_eps, int scaled_channels, float scale, const void* a_rows, int a_stride,
                                const float* A_log, const float* dt_bias, int gate_channels, int beta_col,
                                int beta_heads, float* y, int out_stride, int tokens, int dtype,
                                cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (taps_count < 1 || taps_count > DELTA_MAX_TAPS || ((unit_channels || gate_channels) && unit_dim < 1) ||
      out_stride < channels + gate_channels + beta_heads)
    return (int)cudaErrorInvalidValue;
  // Few tokens: many small blocks a token, so that a decode step fills the GPU; many tokens: a
  // block takes about a thousand channels, since a block that lives for one channel a thread
  // costs more to start than to run.
  const int threads = tokens <= 32 ? 128 : 256;
  const int unit = unit_dim > 0 ? unit_dim : 1;
  const int aim = tokens <= 32 ? 128 : 1024;
  const int chunk = aim >= unit ? (aim / unit) * unit : unit;
  const size_t smem = sizeof(float) * (size_t)chunk;
  const dim3 grid(tokens, (channels + chunk - 1) / chunk);
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(short_conv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    launch_pdl(short_conv_kernel<T>, grid, dim3(threads), smem, stream, (const T*)proj, stride, col0, channels, taps_count,
               taps, state, cu_seqlens, state_slots, num_seqs, unit_channels, unit, unit_eps, scaled_channels,
               scale, (const T*)a_rows, a_stride, A_log, dt_bias, gate_channels, beta_col, beta_heads, y, out_stride,
               chunk);
  });
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// The recurrence. Grid (heads x column parts, requests). A block owns `cols` of the head's dv value
// channels (the columns of S are independent of one another) with P threads to a column: thread
// (j, p) keeps rows p R .. p R + R - 1 of column j of S in registers (R = DK / P rounded up). A
// request's tokens are taken DELTA_CHUNK at a time through two stages of shared memory: while the
// recurrence walks one chunk, token after token (the P threads of a column sit in one warp, so
// nothing block-wide is waited for between tokens), the next chunk's q, k, decay, beta and v are on
// their way (cp.async where the sizes allow 16-byte pieces).
// With one column part to a head the block also norms the head's output over dv, weights, gates and
// stores it; with several, the raw outputs go to `o_raw` and delta_out_kernel finishes them.
// The block of head 0, part 0 also moves the request's convolution state on (nothing reads it here).
//
// conv:  float32 [tokens, conv_stride]: q heads (G x DK) | k heads (G x DK) | v heads (H x dv) |
//        decay (H x DK) | beta (H), as short_conv_kernel leaves them.
// rows:  the projected rows (element type T), raw convolution inputs at in_col (C wide).
#ifndef DELTA_CHUNK
#define DELTA_CHUNK 16
#endif

__device__ __forceinline__ void delta_cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}

template <typename T, int P, int MAX_THREADS>
__global__ void __launch_bounds__(MAX_THREADS) delta_rule_kernel(
    const float* __restrict__ conv, int conv_stride, int C, int G, int H, int dv, int cols, int parts,
    const T* __restrict__ rows, int stride, int in_col, const T* __restrict__ gate_rows, int gate_stride,
    const float* __restrict__ norm_w, float eps, float* __restrict__ S_state, float* __restrict__ conv_state, int K,
    const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, T* __restrict__ out,
    float* __restrict__ o_raw, int vector_loads) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DK = DELTA_DK;
  constexpr int R = (DK + P - 1) / P;
  constexpr int SEG = R + 4;          // a thread's rows, padded so that the P segments fall on different banks
  constexpr int VROW = P * SEG;       // floats of one token's vector of DK
  constexpr int TC = DELTA_CHUNK;
  extern __shared__ __align__(16) float shared[];
  const int stage_floats = TC * (3 * VROW + cols + 4);
  float* os = shared + 2 * stage_floats;  // [TC][cols]
  const int head = blockIdx.x / parts, part = blockIdx.x % parts, seq = blockIdx.y;
  const int col0 = part * cols;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  const int slot = state_slots[seq];
  const int j = threadIdx.x / P, p = threadIdx.x % P;
  const bool live = j < cols && col0 + j < dv;
  const int group = head / (H / G);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

  float S[R];
  float* mine = S_state + (((size_t)slot * H + head) * DK) * dv + col0 + j;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = p * R + i;
    S[i] = (live && r < DK) ? mine[(size_t)r * dv] : 0.f;
  }

  // A stage: q, k, decay [TC][VROW] each, v [TC][cols], beta [TC] (4 floats a token, the first used).
  auto load = [&](int stage, int t0) {
    float* qs = shared + stage * stage_floats;
    float* ks = qs + TC * VROW;
    float* gs = ks + TC * VROW;
    float* vs = gs + TC * VROW;
    float* bs = vs + TC * cols;
    const int n = min(TC, end - t0);
    if (vector_loads) {
      constexpr int PIECES = DK / 4;
      for (int idx = threadIdx.x; idx < n * PIECES; idx += blockDim.x) {
        const int tok = idx / PIECES, i = 4 * (idx % PIECES);
        const float* src = conv + (size_t)(t0 + tok) * conv_stride;
        const int at = tok * VROW + i + (i / R) * 4;
        delta_cp_async16(qs + at, src + group * DK + i);
        delta_cp_async16(ks + at, src + (G + group) * DK + i);
        delta_cp_async16(gs + at, src + C + head * DK + i);
      }
      for (int idx = threadIdx.x; idx < n * (cols / 4); idx += blockDim.x) {
        const int tok = idx / (cols / 4), c = 4 * (idx % (cols / 4));
        delta_cp_async16(vs + tok * cols + c, conv + (size_t)(t0 + tok) * conv_stride + 2 * G * DK + head * dv + col0 + c);
      }
    } else {
      for (int idx = threadIdx.x; idx < n * DK; idx += blockDim.x) {
        const int tok = idx / DK, i = idx % DK;
        const float* src = conv + (size_t)(t0 + tok) * conv_stride;
        const int at = tok * VROW + i + (i / R) * 4;
        qs[at] = src[group * DK + i];
        ks[at] = src[(G + group) * DK + i];
        gs[at] = src[C + head * DK + i];
      }
      for (int idx = threadIdx.x; idx < n * cols; idx += blockDim.x) {
        const int tok = idx / cols, c = idx % cols;
        vs[tok * cols + c] = col0 + c < dv ? conv[(size_t)(t0 + tok) * conv_stride + 2 * G * DK + head * dv + col0 + c] : 0.f;
      }
    }
    for (int tok = threadIdx.x; tok < n; tok += blockDim.x)
      bs[4 * tok] = conv[(size_t)(t0 + tok) * conv_stride + C + H * DK + head];
  };

  if (end > begin) load(0, begin);
  asm volatile("cp.async.commit_group;\n" ::);
  int stage = 0;
  for (int t0 = begin; t0 < end; t0 += TC, stage ^= 1) {
    const int n = min(TC, end - t0);
    if (t0 + TC < end) load(stage ^ 1, t0 + TC);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();  // this chunk is in shared memory
    const float* qs = shared + stage * stage_floats;
    const float* ks = qs + TC * VROW;
    const float* gs = ks + TC * VROW;
    const float* vs = gs + TC * VROW;
    const float* bs = vs + TC * cols;
#pragma unroll 2
    for (int tok = 0; tok < n; ++tok) {
      const float* gt = gs + tok * VROW + p * SEG;
      const float* kt = ks + tok * VROW + p * SEG;
      const float* qt = qs + tok * VROW + p * SEG;
      float dot;
      if constexpr (R % 4 == 0 && DK % P == 0) {
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 g4 = *reinterpret_cast<const float4*>(gt + i), k4 = *reinterpret_cast<const float4*>(kt + i);
          S[i] *= g4.x, S[i + 1] *= g4.y, S[i + 2] *= g4.z, S[i + 3] *= g4.w;
          d0 += S[i] * k4.x, d1 += S[i + 1] * k4.y, d2 += S[i + 2] * k4.z, d3 += S[i + 3] * k4.w;
        }
        dot = (d0 + d1) + (d2 + d3);
      } else {
        dot = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i)
          if (p * R + i < DK) {
            S[i] *= gt[i];
            dot += S[i] * kt[i];
          }
      }
#pragma unroll
      for (int o = 1; o < P; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = bs[4 * tok] * ((live ? vs[tok * cols + j] : 0.f) - dot);
      float o_j;
      if constexpr (R % 4 == 0 && DK % P == 0) {
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
        for (int i = 0; i < R; i += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kt + i), q4 = *reinterpret_cast<const float4*>(qt + i);
          S[i] += k4.x * u, S[i + 1] += k4.y * u, S[i + 2] += k4.z * u, S[i + 3] += k4.w * u;
          d0 += S[i] * q4.x, d1 += S[i + 1] * q4.y, d2 += S[i + 2] * q4.z, d3 += S[i + 3] * q4.w;
        }
        o_j = (d0 + d1) + (d2 + d3);
      } else {
        o_j = 0.f;
#pragma unroll
        for (int i = 0; i < R; ++i)
          if (p * R + i < DK) {
            S[i] += kt[i] * u;
            o_j += S[i] * qt[i];
          }
      }
#pragma unroll
      for (int o = 1; o < P; o <<= 1) o_j += __shfl_xor_sync(0xffffffffu, o_j, o);
      if (live && p == 0) {
        if (parts == 1) os[tok * cols + j] = o_j;
        else o_raw[(size_t)(t0 + tok) * H * dv + head * dv + col0 + j] = o_j;
      }
    }
    __syncthreads();  // the chunk's outputs are complete, and its stage may be loaded over
    if (parts == 1) {
      for (int tok = warp; tok < n; tok += nwarps) {
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) ss += os[tok * cols + c] * os[tok * cols + c];
        const float r = rsqrtf(warp_sum(ss) / (float)dv + eps);
        const size_t t = t0 + tok;
        for (int c = lane; c < dv; c += 32) {
          const float gate = to_f32(gate_rows[t * gate_stride + head * dv + c]);
          out[t * H * dv + head * dv + c] = from_f32<T>(os[tok * cols + c] * r * norm_w[c] / (1.f + expf(-gate)));
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = p * R + i;
    if (live && r < DK) mine[(size_t)r * dv] = S[i];
  }

  if (blockIdx.x == 0 && K > 1 && end > begin) {
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

// out = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate) per (token, head); a warp each.
template <typename T>
__global__ void delta_out_kernel(const float* __restrict__ o_raw, const T* __restrict__ gate_rows, int gate_stride,
                                 const float* __restrict__ norm_w, float eps, int H, int dv, int total,
                                 T* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= total) return;
  const size_t t = item / H;
  const int head = item % H;
  const float* o = o_raw + t * H * dv + head * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += o[c] * o[c];
  const float r = rsqrtf(warp_sum(ss) / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float gate = to_f32(gate_rows[t * gate_stride + head * dv + c]);
    out[t * H * dv + head * dv + c] = from_f32<T>(o[c] * r * norm_w[c] / (1.f + expf(-gate)));
  }
}

extern "C" int omnia_delta_dk(void) { return DELTA_DK; }

// parts: column parts a head (1: the norm is done in the recurrence kernel; more: o_raw float32
// [tokens, H * dv] is needed). dv must divide into `parts` equal runs of a multiple of 4 columns.
extern "C" int omnia_delta_rule(const float* conv, int conv_stride, int C, int G, int H, int dv, int parts,
                                const void* rows, int stride, int in_col, const void* gate_rows, int gate_stride,
                                const float* norm_w, float eps, float* S_state, float* conv_state, int taps_count,
                                const int* cu_seqlens, const int* state_slots, int num_seqs, int tokens, void* out,
                                float* o_raw, int dtype, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (G < 1 || H % G != 0 || dv < 1 || dv > 1024 || taps_count < 1 || taps_count > DELTA_MAX_TAPS ||
      C != 2 * G * DELTA_DK + H * dv || conv_stride < C + H * DELTA_DK + H || parts < 1 || dv % parts != 0 ||
      (parts > 1 && (o_raw == nullptr || (dv / parts) % 4 != 0)))
    return (int)cudaErrorInvalidValue;
  const int cols = dv / parts;
  const dim3 grid(H * parts, num_seqs);
#define OMNIA_DELTA_LAUNCH(P, MAX_THREADS)                                                                        \
  do {                                                                                                            \
    constexpr int R = (DELTA_DK + P - 1) / P;                                                                     \
    constexpr int SEG = R + 4;                                                                                    \
    const int vector_loads = R % 4 == 0 && DELTA_DK % P == 0 && conv_stride % 4 == 0 && C % 4 == 0 &&             \
                             cols % 4 == 0 && dv % 4 == 0 && (2 * G * DELTA_DK) % 4 == 0;                         \
    const size_t smem = sizeof(float) * ((size_t)2 * DELTA_CHUNK * (3 * P * SEG + cols + 4) + DELTA_CHUNK * cols); \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(delta_rule_kernel<T, P, MAX_THREADS>,                            \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return (int)cudaGetLastError();                                                                             \
    launch_pdl(delta_rule_kernel<T, P, MAX_THREADS>, grid, dim3((cols * P + 31) / 32 * 32), smem, stream, conv,   \
               conv_stride, C, G, H, dv, cols, parts, (const T*)rows, stride, in_col, (const T*)gate_rows,        \
               gate_stride, norm_w, eps, S_state, conv_state, taps_count, cu_seqlens, state_slots, (T*)out, o_raw, \
               vector_loads);                                                                                     \
  } while (0)
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (cols * 4 <= 128) OMNIA_DELTA_LAUNCH(4, 128);
    else if (cols * 4 <= 512) OMNIA_DELTA_LAUNCH(4, 512);
    else if (cols * 4 <= 1024) OMNIA_DELTA_LAUNCH(4, 1024);
    else if (cols * 2 <= 1024) OMNIA_DELTA_LAUNCH(2, 1024);
    else OMNIA_DELTA_LAUNCH(1, 1024);
  });
#undef OMNIA_DELTA_LAUNCH
  int code = OMNIA_LAUNCH_RESULT();
  if (code != 0 || parts == 1) return code;
  const int total = tokens * H;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(delta_out_kernel<T>, dim3((total + 3) / 4), dim3(128), 0, stream,
                                          (const float*)o_raw, (const T*)gate_rows, gate_stride, norm_w, eps, H, dv,
                                          total, (T*)out)));
  return OMNIA_LAUNCH_RESULT();
}
