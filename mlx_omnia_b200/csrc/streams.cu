// The residual as several streams (hyper-connections), the grouped RMS norm and the token shift:
// the two kernels a pre-norm block with these options runs around each of its branches.
//
//   enter:  u = sum_s a[s] x_s;  n = grouped_rms(u) * w;  h = n + (n_prev - n) * mu     (mu optional)
//   leave:  x_t <- sum_s M[s, t] x_s + b[t] * y    for all t at once                    (M, b optional: x += y)
//           and, when asked, the entry of the branch that follows (without a shift) from the new x
//
// x is float32 [tokens, S, D] (S = 1: the plain residual). One block per token, or several that
// take whole norm groups each when the step has few tokens. All arithmetic is
// float32; only h and y have the engine's element type. The order of every sum depends on the
// sizes alone, never on how a batch was cut.
//
// Token shift: n_prev is the un-shifted n of the token before in the same request. For the first
// token of a request's portion it is read from the request's state slot (`prev`, zeros for a fresh
// request); for any other it is computed again from the row before. The last token of a portion
// leaves its n in `last` [requests, D], and the block's *leave* kernel copies that into the slot:
// a portion's first token reads the slot while its last one would write it, so the write waits
// for the next kernel.
#include "common.cuh"

#define OMNIA_MAX_STREAMS 8

// The request of token t: the last s with cu_seqlens[s] <= t.
__device__ __forceinline__ int request_of(const int* __restrict__ cu_seqlens, int num_seqs, int t) {
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// A block's share of a row: with gridDim.y blocks a token, block y takes whole norm groups
// [g_lo, g_hi) = columns [lo, hi). A step of few tokens is spread over many blocks this way; a
// step of many has one block a token.
struct RowShare {
  int g_lo, g_hi, lo, hi;
};
__device__ __forceinline__ RowShare row_share(int D, int groups) {
  const int per = (groups + gridDim.y - 1) / gridDim.y;
  const int gs = D / groups;
  RowShare r;
  r.g_lo = min(groups, (int)blockIdx.y * per);
  r.g_hi = min(groups, r.g_lo + per);
  r.lo = r.g_lo * gs;
  r.hi = r.g_hi * gs;
  return r;
}

// h = grouped_rms(u0) * w over the block's groups, shifted towards the row before when mu is given
// (that row is u1, normed here too, or `prev_row` as it stands). u0, u1: shared memory, column
// `share.lo` first; part: shared [2][32]. The row pointers are of whole rows. A team of W warps
// per group; teams take the groups in turn; every sum in a fixed order.
template <typename T>
__device__ __forceinline__ void grouped_norm_store(const float* u0, const float* u1, int D, int groups, RowShare share,
                                                   const float* __restrict__ w, float eps,
                                                   const float* __restrict__ mu, bool from_state,
                                                   const float* __restrict__ prev_row, float* __restrict__ last_row,
                                                   T* __restrict__ h_row, float (*part)[32]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int mine = share.g_hi - share.g_lo;
  const int W = mine > 0 && mine < nwarps ? nwarps / mine : 1;
  const int teams = nwarps / W;
  const int team = warp / W, wi = warp % W;
  const int gs = D / groups;
  for (int g0 = share.g_lo; g0 < share.g_hi; g0 += teams) {
    const int g = g0 + team;
    const bool active = team < teams && g < share.g_hi;
    float s0 = 0.f, s1 = 0.f;
    if (active) {
      for (int i = g * gs + wi * 32 + lane; i < (g + 1) * gs; i += W * 32) {
        s0 += u0[i - share.lo] * u0[i - share.lo];
        if (mu != nullptr) s1 += u1[i - share.lo] * u1[i - share.lo];
      }
    }
    s0 = warp_sum(s0);
    s1 = warp_sum(s1);
    __syncthreads();
    if (lane == 0) part[0][warp] = s0, part[1][warp] = s1;
    __syncthreads();
    if (!active) continue;
    float t0 = 0.f, t1 = 0.f;
    for (int j = 0; j < W; ++j) t0 += part[0][team * W + j], t1 += part[1][team * W + j];
    const float r0 = rsqrtf(t0 / (float)gs + eps), r1 = rsqrtf(t1 / (float)gs + eps);
    for (int i = g * gs + wi * 32 + lane; i < (g + 1) * gs; i += W * 32) {
      const float n = u0[i - share.lo] * r0 * w[i];
      float out = n;
      if (mu != nullptr) {
        const float before = from_state ? prev_row[i] : u1[i - share.lo] * r1 * w[i];
        out = n + (before - n) * mu[i];
        if (last_row != nullptr) last_row[i] = n;
      }
      h_row[i] = from_f32<T>(out);
    }
  }
}

template <typename T>
__global__ void streams_enter_kernel(const float* __restrict__ xs, const float* __restrict__ coef, int S, int D,
                                     const float* __restrict__ w, float eps, int groups,
                                     const float* __restrict__ mu, const float* __restrict__ prev,
                                     float* __restrict__ last, const int* __restrict__ cu_seqlens,
                                     const int* __restrict__ state_slots, int num_seqs, T* __restrict__ h,
                                     float* __restrict__ sum_out, int share_floats) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float rows[];  // the block's columns of u of this token, and of the token before
  __shared__ float part[2][32];
  const int t = blockIdx.x;
  const RowShare share = row_share(D, groups);
  if (share.lo >= share.hi) return;
  float a[OMNIA_MAX_STREAMS];
#pragma unroll
  for (int s = 0; s < OMNIA_MAX_STREAMS; ++s) a[s] = s < S ? (coef ? coef[s] : 1.f) : 0.f;

  int seq = 0, from_state = 0, is_last = 0;
  if (mu != nullptr) {
    seq = request_of(cu_seqlens, num_seqs, t);
    from_state = t == cu_seqlens[seq];
    is_last = t + 1 == cu_seqlens[seq + 1];
  }
  const bool again = mu != nullptr && !from_state;  // the row before is normed again
  float* u0 = rows;
  float* u1 = rows + share_floats;
  // All of a thread's loads are asked for before the first is used: the stream count is a loop
  // bound the compiler knows, and four elements go side by side.
  for (int i0 = share.lo + threadIdx.x; i0 < share.hi; i0 += 4 * blockDim.x) {
    float v[4] = {0.f, 0.f, 0.f, 0.f}, p[4] = {0.f, 0.f, 0.f, 0.f};
    float x[4][OMNIA_MAX_STREAMS], xp[4][OMNIA_MAX_STREAMS];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = i0 + e * blockDim.x;
#pragma unroll
      for (int s = 0; s < OMNIA_MAX_STREAMS; ++s) {
        x[e][s] = (s < S && i < share.hi) ? xs[((size_t)t * S + s) * D + i] : 0.f;
        xp[e][s] = (again && s < S && i < share.hi) ? xs[((size_t)(t - 1) * S + s) * D + i] : 0.f;
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = i0 + e * blockDim.x;
#pragma unroll
      for (int s = 0; s < OMNIA_MAX_STREAMS; ++s) v[e] += a[s] * x[e][s], p[e] += a[s] * xp[e][s];
      if (i < share.hi) {
        u0[i - share.lo] = v[e];
        u1[i - share.lo] = p[e];
        if (sum_out != nullptr) sum_out[(size_t)t * D + i] = v[e];
      }
    }
  }
  __syncthreads();
  const float* prev_row = (mu != nullptr && from_state) ? prev + (size_t)state_slots[seq] * D : nullptr;
  grouped_norm_store<T>(u0, u1, D, groups, share, w, eps, mu, from_state, prev_row,
                        is_last ? last + (size_t)seq * D : nullptr, h + (size_t)t * D, part);
}

// How many blocks share a token's row: steps of few tokens are spread over the norm's groups.
static int blocks_per_row(int tokens, int groups) {
  if (tokens > 32 || groups <= 1) return 1;
  return groups < 16 ? groups : 16;
}

extern "C" int omnia_streams_enter(const float* xs, const float* coef, int streams, int width, const float* w,
                                   float eps, int groups, const float* mu, const float* prev, float* last,
                                   const int* cu_seqlens, const int* state_slots, int num_seqs, void* h,
                                   float* sum_out, int tokens, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (streams < 1 || streams > OMNIA_MAX_STREAMS || groups < 1 || width % groups != 0) return (int)cudaErrorInvalidValue;
  const int by = blocks_per_row(tokens, groups);
  const int share_floats = (groups + by - 1) / by * (width / groups);
  const size_t smem = 2 * sizeof(float) * (size_t)share_floats;
  const int threads = share_floats >= 1024 ? 256 : 128;
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(streams_enter_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    launch_pdl(streams_enter_kernel<T>, dim3(tokens, by), dim3(threads), smem, stream, xs, coef, streams, width, w, eps,
               groups, mu, prev, last, cu_seqlens, state_slots, num_seqs, (T*)h, sum_out, share_floats);
  });
  return OMNIA_LAUNCH_RESULT();
}

// Blocks x = 0 .. tokens-1 update a token's streams; blocks x = tokens .. tokens+commits-1 copy a
// request's `last` row into its state slot (see the top of the file). Block y of a row takes the
// columns of whole groups of the norm that follows (`next_groups`; any even cut when none follows).
template <typename T>
__global__ void streams_leave_kernel(float* __restrict__ xs, const T* __restrict__ y, const float* __restrict__ mix,
                                     const float* __restrict__ outc, int S, int D, int tokens,
                                     const float* __restrict__ last, float* __restrict__ prev,
                                     const int* __restrict__ state_slots, const float* __restrict__ next_coef,
                                     const float* __restrict__ next_w, float next_eps, int next_groups,
                                     T* __restrict__ next_h) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float rows[];  // the block's columns when the next branch is entered here
  __shared__ float part[2][32];
  const int t = blockIdx.x;
  const RowShare share = row_share(D, next_groups);
  if (share.lo >= share.hi) return;
  if (t >= tokens) {
    const int seq = t - tokens;
    float* to = prev + (size_t)state_slots[seq] * D;
    for (int i = share.lo + threadIdx.x; i < share.hi; i += blockDim.x) to[i] = last[(size_t)seq * D + i];
    return;
  }
  __shared__ float m[OMNIA_MAX_STREAMS * OMNIA_MAX_STREAMS + 2 * OMNIA_MAX_STREAMS];
  if (threadIdx.x < S * S) m[threadIdx.x] = mix ? mix[threadIdx.x] : 1.f;
  if (threadIdx.x < S) {
    m[OMNIA_MAX_STREAMS * OMNIA_MAX_STREAMS + threadIdx.x] = outc ? outc[threadIdx.x] : 1.f;
    m[OMNIA_MAX_STREAMS * OMNIA_MAX_STREAMS + OMNIA_MAX_STREAMS + threadIdx.x] = next_coef ? next_coef[threadIdx.x] : 1.f;
  }
  __syncthreads();
  for (int i = share.lo + threadIdx.x; i < share.hi; i += blockDim.x) {
    float old[OMNIA_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < OMNIA_MAX_STREAMS; ++s)
      if (s < S) old[s] = xs[((size_t)t * S + s) * D + i];
    const float branch = to_f32(y[(size_t)t * D + i]);
    float next_u = 0.f;
#pragma unroll
    for (int to = 0; to < OMNIA_MAX_STREAMS; ++to) {
      if (to >= S) break;
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < OMNIA_MAX_STREAMS; ++s)
        if (s < S) v += m[s * S + to] * old[s];
      const float fresh = v + m[OMNIA_MAX_STREAMS * OMNIA_MAX_STREAMS + to] * branch;
      xs[((size_t)t * S + to) * D + i] = fresh;
      next_u += m[OMNIA_MAX_STREAMS * OMNIA_MAX_STREAMS + OMNIA_MAX_STREAMS + to] * fresh;
    }
    if (next_h != nullptr) rows[i - share.lo] = next_u;
  }
  if (next_h == nullptr) return;
  // The branch after this one reads the new streams: its entry (sum, grouped norm, weight; no
  // token shift) is done here, while the row is still at hand.
  __syncthreads();
  grouped_norm_store<T>(rows, rows, D, next_groups, share, next_w, next_eps, nullptr, false, nullptr, nullptr,
                        next_h + (size_t)t * D, part);
}

extern "C" int omnia_streams_leave(float* xs, const void* y, const float* mix, const float* outc, int streams,
                                   int width, int tokens, const float* last, float* prev, const int* state_slots,
                                   int commits, const float* next_coef, const float* next_w, float next_eps,
                                   int next_groups, void* next_h, int dtype, cudaStream_t stream) {
  if (tokens + commits == 0) return 0;
  if (streams < 1 || streams > OMNIA_MAX_STREAMS || (mix == nullptr && streams != 1)) return (int)cudaErrorInvalidValue;
  if (next_h != nullptr && (next_groups < 1 || width % next_groups != 0 || next_w == nullptr)) return (int)cudaErrorInvalidValue;
  // Without a norm to follow, the row is cut as evenly as its width allows.
  int cut = next_groups;
  if (next_h == nullptr) {
    cut = 1;
    for (int c = 16; c >= 2; c >>= 1)
      if (width % c == 0) { cut = c; break; }
  }
  const int by = blocks_per_row(tokens, cut);
  const int share_floats = (cut + by - 1) / by * (width / cut);
  const size_t smem = next_h != nullptr ? sizeof(float) * (size_t)share_floats : 0;
  const int threads = share_floats >= 1024 ? 256 : 128;
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(streams_leave_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    launch_pdl(streams_leave_kernel<T>, dim3(tokens + commits, by), dim3(threads), smem, stream, xs, (const T*)y, mix,
               outc, streams, width, tokens, last, prev, state_slots, next_coef, next_w, next_eps, cut, (T*)next_h);
  });
  return OMNIA_LAUNCH_RESULT();
}

// x_s = table[id] * multiplier for every stream s: the residual streams at their start.
template <typename T>
__global__ void embed_streams_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ xs,
                                     int S, int D, int vocab, float multiplier, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(err, OMNIA_ERR_TOKEN_ID);
    id = 0;
  }
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = to_f32(table[(size_t)id * D + i]) * multiplier;
    for (int s = 0; s < S; ++s) xs[((size_t)t * S + s) * D + i] = v;
  }
}

extern "C" int omnia_embed_streams(const int* ids, const void* table, float* xs, int tokens, int streams, int width,
                                   int vocab, float multiplier, int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(embed_streams_kernel<T>, tokens, 256, 0, stream, ids, (const T*)table, xs,
                                          streams, width, vocab, multiplier, err)));
  return OMNIA_LAUNCH_RESULT();
}
