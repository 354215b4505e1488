// Attention over a latent cache: one row [rank | rot] per position, shared by all heads.
//
// A position's row holds the normed low-rank latent c (rank wide) and one rotated key part (rot
// wide). With the key and value expansions folded into the query and the output
// (q_lat = W_uk^T q_plain, out = W_uv o_lat), head h scores position j as
//   s = (q_lat[h] . c_j + q_rot[h] . r_j) * scale
// and its output in latent space is o_lat[h] = sum_j p_j c_j: every head reads the same rows, and
// the rows are both keys and values. The softmax's denominator also holds exp(sink[h]) when a sink
// is given: a term without key and value, not scaled. The output is multiplied by
// sigmoid(gate[t, h]) when a gate is given.
//
// Two kernels: the one that prepares a step's rows (norm of the latent, rotation of the shared key
// part and of the queries' rotated parts, cache write), and the attention itself.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Per token: c = rms(down[:rank]) * w -> cache[slot, :rank]; the last `rot` columns of the down
// projection, rotated, -> cache[slot, rank:]; and the last `rot` of every query head rotated in
// place in the projected rows. Rotation: the first rot_dims dims in pairs (2i, 2i + 1), angle
// position * inv_freq[i] in float32; dims beyond rot_dims pass unchanged.
template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ proj, int stride, int q_col, int heads, int q_dim,
                                      int down_col, int rank, int rot, const float* __restrict__ w, float eps,
                                      const float* __restrict__ inv_freq, int rot_dims,
                                      const int* __restrict__ positions, const long long* __restrict__ slot_mapping,
                                      T* __restrict__ cache, long long total_slots, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  T* row = proj + (size_t)t * stride;
  const float pos = (float)positions[t];
  const long long slot = slot_mapping ? slot_mapping[t] : -1;
  const bool store = slot >= 0;  // a padding row of a captured step has slot -1
  if (slot >= total_slots) {
    if (threadIdx.x == 0) atomicOr(err, OMNIA_ERR_SLOT);
    return;
  }
  T* to = cache + (size_t)(store ? slot : 0) * (rank + rot);
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f32(row[down_col + i]);
    ss += v * v;
  }
  const float r = rsqrtf(block_sum(ss, scratch) / (float)rank + eps);
  if (store)
    for (int i = threadIdx.x; i < rank; i += blockDim.x) to[i] = from_f32<T>(to_f32(row[down_col + i]) * r * w[i]);
  // Rotations: job 0 is the shared key part, jobs 1 .. heads the queries' rotated parts.
  const int half = rot_dims / 2;
  for (int item = threadIdx.x; item < (heads + 1) * half; item += blockDim.x) {
    const int job = item / half, i = item % half;
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    T* at = job == 0 ? row + down_col + rank : row + q_col + (size_t)(job - 1) * q_dim + (q_dim - rot);
    const float a = to_f32(at[2 * i]), b = to_f32(at[2 * i + 1]);
    const T ra = from_f32<T>(a * c - b * s), rb = from_f32<T>(b * c + a * s);
    if (job == 0) {
      if (store) to[rank + 2 * i] = ra, to[rank + 2 * i + 1] = rb;
    } else {
      at[2 * i] = ra, at[2 * i + 1] = rb;
    }
  }
  if (store)
    for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) to[rank + i] = row[down_col + rank + i];
}

extern "C" int omnia_latent_prepare(void* proj, int stride, int q_col, int heads, int q_dim, int down_col, int rank,
                                    int rot, const float* w, float eps, const float* inv_freq, int rot_dims,
                                    const int* positions, const long long* slot_mapping, void* cache,
                                    long long total_slots, int tokens, int dtype, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (rot_dims % 2 != 0 || rot_dims > rot || rot > q_dim || rank < 1) return (int)cudaErrorInvalidValue;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(latent_prepare_kernel<T>, tokens, 128, 0, stream, (T*)proj, stride, q_col,
                                          heads, q_dim, down_col, rank, rot, w, eps, inv_freq, rot_dims, positions,
                                          slot_mapping, (T*)cache, total_slots, err)));
  return OMNIA_LAUNCH_RESULT();
}

// ---------------------------------------------------------------------------------
// One warp per (token, head), any batch shape and element type. Keys are visited 32 at a time
// from the lowest visible position; a lane scores one key (a full dot product in float32), the
// chunk's softmax statistics are merged online, and for the output a lane owns the latent dims
// lane, lane + 32, ... The order of all additions depends on the token's position and window alone.
#define LATENT_MAX_ACC 16  // rank <= 512

template <typename T>
__global__ void latent_attention_kernel(const T* __restrict__ q_lat, long long q_lat_stride_h, long long q_lat_stride_t,
                                        const T* __restrict__ q_rot, long long q_rot_stride_h, long long q_rot_stride_t,
                                        const T* __restrict__ cache, const int* __restrict__ block_table,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                                        const float* __restrict__ sink, const T* __restrict__ gate, int gate_stride,
                                        T* __restrict__ out, long long out_stride_h, long long out_stride_t,
                                        int num_seqs, int max_pages, int num_pages, int heads, int rank, int rot,
                                        int page_size, int window, float scale, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float qs_all[];  // [4][rank + rot]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * 4 + warp;
  if (head >= heads) return;
  const int width = rank + rot;
  float* qs = qs_all + warp * width;
  int lo_s = 0, hi_s = num_seqs - 1;
  while (lo_s < hi_s) {
    const int mid = (lo_s + hi_s + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo_s = mid; else hi_s = mid - 1;
  }
  const int seq = lo_s;
  const int pos = positions[t];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const T* ql = q_lat + head * q_lat_stride_h + t * q_lat_stride_t;
  const T* qr = q_rot + head * q_rot_stride_h + t * q_rot_stride_t;
  for (int i = lane; i < rank; i += 32) qs[i] = to_f32(ql[i]) * scale;
  for (int i = lane; i < rot; i += 32) qs[rank + i] = to_f32(qr[i]) * scale;
  __syncwarp();

  // The sink is one more term of the denominator: the running maximum starts at it and the sum at 1.
  float m = sink ? sink[head] : -INFINITY, l = sink ? 1.f : 0.f;
  float acc[LATENT_MAX_ACC];
#pragma unroll
  for (int k = 0; k < LATENT_MAX_ACC; ++k) acc[k] = 0.f;
  const int* table = block_table + (size_t)seq * max_pages;

  for (int base = first; base <= pos; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    long long krow = -1;
    if (j <= pos) {
      const int page = table[j / page_size];
      if (page < 0 || page >= num_pages) {
        atomicOr(err, OMNIA_ERR_PAGE);
      } else {
        krow = (long long)page * page_size + j % page_size;
        const T* kp = cache + krow * width;
        float dot = 0.f;
        for (int i = 0; i < width; ++i) dot += qs[i] * to_f32(kp[i]);
        s = dot;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float alpha = expf(m - m_new);
    const float p = s == -INFINITY ? 0.f : expf(s - m_new);
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int k = 0; k < LATENT_MAX_ACC; ++k) acc[k] *= alpha;
    const int count = min(32, pos - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long vr = __shfl_sync(0xffffffffu, krow, jj);
      if (vr < 0) continue;
      const T* vp = cache + vr * width;
#pragma unroll
      for (int k = 0; k < LATENT_MAX_ACC; ++k) {
        const int i = lane + 32 * k;
        if (i < rank) acc[k] += pj * to_f32(vp[i]);
      }
    }
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
  if (gate != nullptr) inv *= 1.f / (1.f + expf(-to_f32(gate[(size_t)t * gate_stride + head])));
  T* orow = out + head * out_stride_h + t * out_stride_t;
#pragma unroll
  for (int k = 0; k < LATENT_MAX_ACC; ++k) {
    const int i = lane + 32 * k;
    if (i < rank) orow[i] = from_f32<T>(acc[k] * inv);
  }
}

extern "C" int omnia_latent_attention(const void* q_lat, long long q_lat_stride_h, long long q_lat_stride_t,
                                      const void* q_rot, long long q_rot_stride_h, long long q_rot_stride_t,
                                      const void* cache, const int* block_table, const int* cu_seqlens,
                                      const int* positions, const float* sink, const void* gate, int gate_stride,
                                      void* out, long long out_stride_h, long long out_stride_t, int tokens,
                                      int num_seqs, int max_pages, int num_pages, int heads, int rank, int rot,
                                      int page_size, int window, float scale, int dtype, int* err,
                                      cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (rank < 1 || rank > 32 * LATENT_MAX_ACC || rot < 0 || heads < 1) return (int)cudaErrorInvalidValue;
  const dim3 grid(tokens, (heads + 3) / 4);
  const size_t smem = 4 * sizeof(float) * (size_t)(rank + rot);
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(latent_attention_kernel<T>, grid, 128, smem, stream, (const T*)q_lat,
                                          q_lat_stride_h, q_lat_stride_t, (const T*)q_rot, q_rot_stride_h,
                                          q_rot_stride_t, (const T*)cache, block_table, cu_seqlens, positions, sink,
                                          (const T*)gate, gate_stride, (T*)out, out_stride_h, out_stride_t, num_seqs,
                                          max_pages, num_pages, heads, rank, rot, page_size, window, scale, err)));
  return OMNIA_LAUNCH_RESULT();
}
