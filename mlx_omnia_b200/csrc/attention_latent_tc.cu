// Attention over a latent cache in bfloat16 on the tensor cores (mma.sync m16n8k16, float32
// accumulation and softmax), compiled for one latent width and one rotated width:
//   -DLATENT_RANK=r  (a multiple of 64)   -DLATENT_ROT=d  (r + d a multiple of 32)
//   -DLATENT_ROW_GROUPS=g  (1, 2 or 4: a block owns 16 g rows)
// See attention_latent.cu for what is computed. A cache row [rank | rot] is a key as a whole and
// a value in its first `rank` numbers, the same for every head; so the rows of a tile are (token,
// head) pairs in the order they lie in memory, row R of a request's step being token R / heads,
// head R % heads, and one key tile fetched from the cache serves them all.
//
// A block of 4 g warps owns 16 g rows and walks the keys its rows can see, 32 at a time, through a
// cp.async double buffer. Warp (row group, column quarter): scores of its 16 rows against 8 of the
// tile's keys; the row maxima of the four quarters meet in shared memory, the weights P go there as
// bfloat16; then each warp adds P V for its quarter of the latent columns. The key range may be cut
// into `splits` chunks (aligned to absolute positions) that separate blocks walk; each then leaves
// its unnormalised accumulator, maximum and sum in a workspace, and a second kernel merges a row's
// chunks in ascending order. The sink and the gate are applied where the row is finished. Keys
// outside a block's range are zero-filled in shared memory and never read from the cache.
#include "common.cuh"

#ifndef LATENT_RANK
#define LATENT_RANK 512
#endif
#ifndef LATENT_ROT
#define LATENT_ROT 64
#endif
#ifndef LATENT_ROW_GROUPS
#define LATENT_ROW_GROUPS 2
#endif

namespace {

typedef __nv_bfloat16 bf16;
constexpr int RANK = LATENT_RANK, ROT = LATENT_ROT, WIDTH = RANK + ROT;
constexpr int ROW = WIDTH + 8;          // shared-memory row stride (elements): odd in 16-byte units
constexpr int KSTEPS = WIDTH / 16;
constexpr int RG = LATENT_ROW_GROUPS, CW = 4;
constexpr int BM = 16 * RG, BN = 32;
constexpr int THREADS = 32 * RG * CW;
constexpr int COLS = RANK / CW;         // latent columns a warp accumulates
constexpr int NT_O = COLS / 8;
constexpr int PROW = BN + 8;
constexpr int CHUNKS = WIDTH / 8;       // 16-byte chunks of a row
constexpr float LOG2E = 1.4426950408889634f;
static_assert(RANK % 64 == 0 && WIDTH % 32 == 0, "latent width: rank a multiple of 64, rank + rot of 32");
static_assert(RG == 1 || RG == 2 || RG == 4, "row groups");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned* r, const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

struct Args {
  const bf16* q_lat; long long q_lat_stride_h, q_lat_stride_t;   // [heads, tokens, RANK]
  const bf16* q_rot; long long q_rot_stride_h, q_rot_stride_t;   // [tokens, heads, ROT]
  const bf16* cache;            // [num_pages * page_size, WIDTH]
  const int* block_table;       // [num_seqs, max_pages]
  const int* cu_seqlens;        // [num_seqs + 1]
  const int* seq_lens;          // [num_seqs] positions held after this step
  const float* sink;            // [heads] or null
  const bf16* gate; int gate_stride;  // gate[t * gate_stride + h], or null
  bf16* out; long long out_stride_h, out_stride_t;               // [heads, tokens, RANK]
  float* part_o; float* part_ml;  // [rows, splits, RANK], [rows, splits, 2] when splits > 1
  int max_pages, num_pages, heads, page_size, window, splits, chunk;
  float scale;
  int* err;
};

// The finished row: the sink joins the denominator, the gate multiplies. m is in natural units.
__device__ __forceinline__ float finish_factor(float m, float l, const float* sink, const bf16* gate, int gate_stride,
                                               int token, int head) {
  if (sink != nullptr) {
    const float s = sink[head];
    const float top = fmaxf(m, s);
    const float keep = m == -INFINITY ? 0.f : expf(m - top);
    l = l * keep + expf(s - top);
    l = keep / l;                       // the accumulator is relative to m
  } else {
    l = l > 0.f ? 1.f / l : 0.f;
  }
  if (gate != nullptr) l *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)token * gate_stride + head])));
  return l;
}

__global__ void __launch_bounds__(THREADS) latent_attention_tc_kernel(const Args a) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);     // [BM][ROW]
  bf16* ks = qs + BM * ROW;                         // [2][BN][ROW]
  bf16* ps = ks + 2 * BN * ROW;                     // [BM][PROW]
  float* smax = reinterpret_cast<float*>(ps + BM * PROW);  // [CW][BM]
  float* ssum = smax + CW * BM;                     // [CW][BM]

  const int seq = blockIdx.z, split = blockIdx.y, rb = blockIdx.x;
  const int t_begin = a.cu_seqlens[seq];
  const int q_len = a.cu_seqlens[seq + 1] - t_begin;
  const int rows = q_len * a.heads;
  const int row0 = rb * BM;
  if (row0 >= rows) return;
  const int H = a.heads;
  const int pos0 = a.seq_lens[seq] - q_len;         // position of the step's first token of this request
  const int last_row = min(row0 + BM, rows) - 1;
  const int first_pos = pos0 + row0 / H, last_pos = pos0 + last_row / H;
  int key_lo = a.window > 0 ? max(0, first_pos - a.window + 1) : 0;
  int key_hi = last_pos;                            // inclusive; -1 for a padding request: no keys
  if (a.splits > 1) {
    key_lo = max(key_lo, split * a.chunk);
    key_hi = min(key_hi, (split + 1) * a.chunk - 1);
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = warp / CW, cw = warp % CW;
  const int mat = lane >> 3;
  const int* table = a.block_table + (size_t)seq * a.max_pages;

  // The block's query rows.
  for (int c = tid; c < BM * CHUNKS; c += THREADS) {
    const int r = c / CHUNKS, ch = c % CHUNKS;
    const int R = row0 + r;
    const bool valid = R < rows;
    const int token = t_begin + (valid ? R / H : 0), head = valid ? R % H : 0;
    const bf16* src = ch < RANK / 8 ? a.q_lat + head * a.q_lat_stride_h + token * a.q_lat_stride_t + ch * 8
                                    : a.q_rot + head * a.q_rot_stride_h + token * a.q_rot_stride_t + (ch - RANK / 8) * 8;
    cp_async16(qs + r * ROW + ch * 8, src, valid);
  }
  auto load_keys = [&](int stage, int key0) {
    bf16* dst = ks + stage * BN * ROW;
    for (int c = tid; c < BN * CHUNKS; c += THREADS) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      const int key = key0 + r;
      bool valid = key >= key_lo && key <= key_hi;
      const bf16* src = a.cache;
      if (valid) {
        const int page = table[key / a.page_size];
        if (page < 0 || page >= a.num_pages) {
          atomicOr(a.err, OMNIA_ERR_PAGE);
          valid = false;
        } else {
          src = a.cache + ((size_t)page * a.page_size + key % a.page_size) * WIDTH + ch * 8;
        }
      }
      cp_async16(dst + r * ROW + ch * 8, src, valid);
    }
  };
  const int tile0 = key_lo & ~(BN - 1);
  if (key_hi >= key_lo) load_keys(0, tile0);
  cp_async_commit();

  // Rows g and g + 8 of the warp's 16: their positions and running statistics.
  const int g = lane >> 2, t4 = lane & 3;
  int row_pos[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int R = row0 + rg * 16 + g + 8 * r;
    row_pos[r] = R < rows ? pos0 + R / H : -1;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  const float sl2 = a.scale * LOG2E;

  int stage = 0;
  for (int key0 = tile0; key0 <= key_hi; key0 += BN, stage ^= 1) {
    cp_async_wait<0>();
    __syncthreads();                                  // this tile has landed; the other stage is free
    if (key0 + BN <= key_hi) load_keys(stage ^ 1, key0 + BN);
    cp_async_commit();
    const bf16* kt = ks + stage * BN * ROW;
    // Scores of 16 rows against the 8 keys of this warp's quarter.
    float s[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of products
#pragma unroll 4
    for (int k2 = 0; k2 < KSTEPS / 2; ++k2) {
      unsigned qa[4], qb[4], b[4];
      ldmatrix_x4(qa, qs + (rg * 16 + (mat & 1) * 8 + (lane & 7)) * ROW + (2 * k2) * 16 + (mat >> 1) * 8);
      ldmatrix_x4(qb, qs + (rg * 16 + (mat & 1) * 8 + (lane & 7)) * ROW + (2 * k2 + 1) * 16 + (mat >> 1) * 8);
      ldmatrix_x4(b, kt + (cw * 8 + (lane & 7)) * ROW + k2 * 32 + mat * 8);
      mma_bf16(s, qa, b[0], b[1]);
      mma_bf16(s_odd, qb, b[2], b[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] += s_odd[e];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key0 + cw * 8 + 2 * t4 + (e & 1);
      const int r = e >> 1;
      const bool seen = key >= key_lo && key <= key_hi && key <= row_pos[r] &&
                        (a.window <= 0 || key > row_pos[r] - a.window);
      if (!seen) s[e] = -INFINITY;
      mx[r] = fmaxf(mx[r], s[e]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      if (t4 == 0) smax[cw * BM + rg * 16 + g + 8 * r] = mx[r];
    }
    __syncthreads();
    float alpha[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = rg * 16 + g + 8 * r;
      const float tile_max = fmaxf(fmaxf(smax[row], smax[BM + row]), fmaxf(smax[2 * BM + row], smax[3 * BM + row]));
      const float m_new = fmaxf(m[r], tile_max);
      base[r] = m_new == -INFINITY ? 0.f : m_new * sl2;
      alpha[r] = m[r] == -INFINITY ? 0.f : exp2f(m[r] * sl2 - base[r]);
      m[r] = m_new;
      l[r] *= alpha[r];
    }
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      p[e] = exp2f(s[e] * sl2 - base[e >> 1]);      // exp2(-inf) = 0 for unseen keys
      l[e >> 1] += p[e];
    }
    *reinterpret_cast<unsigned*>(ps + (rg * 16 + g) * PROW + cw * 8 + 2 * t4) = pack_bf16(p[0], p[1]);
    *reinterpret_cast<unsigned*>(ps + (rg * 16 + g + 8) * PROW + cw * 8 + 2 * t4) = pack_bf16(p[2], p[3]);
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      o[j][0] *= alpha[0], o[j][1] *= alpha[0];
      o[j][2] *= alpha[1], o[j][3] *= alpha[1];
    }
    __syncthreads();
    // o += P V for this warp's quarter of the latent columns.
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      unsigned pa[4];
      ldmatrix_x4(pa, ps + (rg * 16 + (mat & 1) * 8 + (lane & 7)) * PROW + kk * 16 + (mat >> 1) * 8);
#pragma unroll
      for (int j2 = 0; j2 < NT_O / 2; ++j2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, kt + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * ROW + cw * COLS + j2 * 16 + (mat >> 1) * 8);
        mma_bf16(o[2 * j2], pa, b[0], b[1]);
        mma_bf16(o[2 * j2 + 1], pa, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();
  // Row sums: within the quad, then over the four quarters.
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  __syncthreads();
  if (t4 == 0) ssum[cw * BM + rg * 16 + g] = l[0], ssum[cw * BM + rg * 16 + g + 8] = l[1];
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = rg * 16 + g + 8 * r;
    const int R = row0 + row;
    if (R >= rows) continue;
    const float total = ssum[row] + ssum[BM + row] + ssum[2 * BM + row] + ssum[3 * BM + row];
    const int token = t_begin + R / H, head = R % H;
    const float mn = m[r] == -INFINITY ? -INFINITY : m[r] * a.scale;   // natural units
    if (a.splits > 1) {
      const size_t slot = ((size_t)token * H + head) * a.splits + split;
      float* po = a.part_o + slot * RANK + cw * COLS;
#pragma unroll
      for (int j = 0; j < NT_O; ++j)
        *reinterpret_cast<float2*>(po + 8 * j + 2 * t4) = make_float2(o[j][2 * r], o[j][2 * r + 1]);
      if (cw == 0 && t4 == 0) a.part_ml[slot * 2] = mn, a.part_ml[slot * 2 + 1] = total;
    } else {
      const float f = finish_factor(mn, total, a.sink, a.gate, a.gate_stride, token, head);
      bf16* orow = a.out + head * a.out_stride_h + token * a.out_stride_t + cw * COLS;
#pragma unroll
      for (int j = 0; j < NT_O; ++j)
        *reinterpret_cast<unsigned*>(orow + 8 * j + 2 * t4) = pack_bf16(o[j][2 * r] * f, o[j][2 * r + 1] * f);
    }
  }
}

// A block per (token, head) and 128 latent columns: the row's chunks merged in ascending order,
// their weights worked out once, the partial rows read side by side.
#define LATENT_MAX_SPLITS 256
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                    int heads, const float* __restrict__ sink, const bf16* __restrict__ gate,
                                    int gate_stride, bf16* __restrict__ out, long long out_stride_h,
                                    long long out_stride_t) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float weight[LATENT_MAX_SPLITS];
  __shared__ float factor;
  const int row = blockIdx.x;
  const int token = row / heads, head = row % heads;
  const float* ml = part_ml + (size_t)row * splits * 2;
  if (threadIdx.x < 32) {
    float top = -INFINITY;
    for (int c = threadIdx.x; c < splits; c += 32) top = fmaxf(top, ml[2 * c]);
    top = warp_max(top);
    float total = 0.f;
    for (int c = threadIdx.x; c < splits; c += 32) {
      const float w = ml[2 * c] == -INFINITY ? 0.f : expf(ml[2 * c] - top);
      weight[c] = w;
      total += ml[2 * c + 1] * w;
    }
    total = warp_sum(total);
    if (threadIdx.x == 0) factor = finish_factor(top, total, sink, gate, gate_stride, token, head);
  }
  __syncthreads();
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= RANK) return;
  const float* po = part_o + (size_t)row * splits * RANK + i;
  float acc = 0.f;
  int c = 0;
  for (; c + 4 <= splits; c += 4) {
    const float x0 = po[(size_t)c * RANK], x1 = po[(size_t)(c + 1) * RANK], x2 = po[(size_t)(c + 2) * RANK],
                x3 = po[(size_t)(c + 3) * RANK];
    acc += weight[c] * x0;
    acc += weight[c + 1] * x1;
    acc += weight[c + 2] * x2;
    acc += weight[c + 3] * x3;
  }
  for (; c < splits; ++c) acc += weight[c] * po[(size_t)c * RANK];
  out[head * out_stride_h + token * out_stride_t + i] = __float2bfloat16_rn(acc * factor);
}

}  // namespace

extern "C" int omnia_latent_attention_tc_rows(void) { return BM; }

extern "C" int omnia_latent_attention_tc(const void* q_lat, long long q_lat_stride_h, long long q_lat_stride_t,
                                         const void* q_rot, long long q_rot_stride_h, long long q_rot_stride_t,
                                         const void* cache, const int* block_table, const int* cu_seqlens,
                                         const int* seq_lens, const float* sink, const void* gate, int gate_stride,
                                         void* out, long long out_stride_h, long long out_stride_t, float* part_o,
                                         float* part_ml, int tokens, int num_seqs, int max_q_len, int max_pages,
                                         int num_pages, int heads, int page_size, int window, int splits, int chunk,
                                         float scale, int* err, cudaStream_t stream) {
  if (tokens == 0 || num_seqs == 0) return 0;
  if (heads < 1 || splits < 1 || splits > LATENT_MAX_SPLITS || (splits > 1 && (chunk < BN || chunk % BN != 0 || part_o == nullptr))) return (int)cudaErrorInvalidValue;
  if ((q_lat_stride_h | q_lat_stride_t | q_rot_stride_h | q_rot_stride_t | out_stride_h | out_stride_t) % 8 != 0 ||
      ((reinterpret_cast<uintptr_t>(q_lat) | reinterpret_cast<uintptr_t>(q_rot) | reinterpret_cast<uintptr_t>(cache)) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(out) & 3) != 0)
    return (int)cudaErrorInvalidValue;
  Args a;
  a.q_lat = (const bf16*)q_lat, a.q_lat_stride_h = q_lat_stride_h, a.q_lat_stride_t = q_lat_stride_t;
  a.q_rot = (const bf16*)q_rot, a.q_rot_stride_h = q_rot_stride_h, a.q_rot_stride_t = q_rot_stride_t;
  a.cache = (const bf16*)cache, a.block_table = block_table, a.cu_seqlens = cu_seqlens, a.seq_lens = seq_lens;
  a.sink = sink, a.gate = (const bf16*)gate, a.gate_stride = gate_stride;
  a.out = (bf16*)out, a.out_stride_h = out_stride_h, a.out_stride_t = out_stride_t;
  a.part_o = part_o, a.part_ml = part_ml;
  a.max_pages = max_pages, a.num_pages = num_pages, a.heads = heads, a.page_size = page_size, a.window = window;
  a.splits = splits, a.chunk = chunk, a.scale = scale, a.err = err;
  const size_t smem = sizeof(bf16) * ((size_t)BM * ROW + 2 * BN * ROW + BM * PROW) + sizeof(float) * 2 * CW * BM;
  static bool sized = false;
  if (!sized) {
    if (cudaFuncSetAttribute(latent_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    sized = true;
  }
  const dim3 grid(((size_t)max_q_len * heads + BM - 1) / BM, splits, num_seqs);
  launch_pdl(latent_attention_tc_kernel, grid, dim3(THREADS), smem, stream, a);
  int code = OMNIA_LAUNCH_RESULT();
  if (code != 0 || splits == 1) return code;
  launch_pdl(latent_merge_kernel, dim3(tokens * heads, (RANK + 127) / 128), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml,
             splits, heads, sink, (const bf16*)gate, gate_stride, (bf16*)out, out_stride_h, out_stride_t);
  return OMNIA_LAUNCH_RESULT();
}
