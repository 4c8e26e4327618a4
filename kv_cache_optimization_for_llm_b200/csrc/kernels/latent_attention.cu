// Attention whose keys and values are up-projections of a small latent per token: only the
// latent c (RMS-normed, `rank` wide) and one rotated key part shared by all heads (`rot` wide)
// are cached, as one row of Dc = rank + rot elements per token in the paged cache.
//
// The up-projections are moved to the query side: with k_h = U_h c the score q.k_h equals
// (U_h^T q).c, so every head attends with an "absorbed" query [U_h^T q_plain | q_rot] over the
// same cached rows, the weighted sum of the latents comes out [rank] wide per head and the
// value up-projection is applied to it afterwards.  Three kernels:
//   latent_prep       per token: RMS norm of the query latent, RMS norm of the key/value latent,
//                     interleaved rotary encoding of the shared key part, cache write
//   head_gemm         a product per head, out[t, h, :] = W[h] . in[t, h, :]  (absorbs the queries,
//                     and up-projects the attended latents)
//   latent_attention  causal softmax attention of all heads over the cached rows, with a sink:
//                     the denominator also holds exp(sink_h), a key without a value
// Scores, softmax weights, sums and angles are float32.  Keys are walked in chunks of 32 by
// absolute position, so a token's result does not depend on how its request was cut into steps,
// on the rest of the batch or on where its pages lie.
#include "common.cuh"

#include <math_constants.h>

// ---------------------------------------------------------------- prep
// d_in [T, ld]: the query latent at column 0 (q_rank wide), the key/value latent at column
// kv_off (rank wide) followed by the shared key part (rot wide).
// cq[t] = rms(d_in[t, :q_rank]) * wq;  page row = [ rms(latent) * wkv | rotate(shared part) ].
// Rotation: pairs (2i, 2i + 1) for i < rdims / 2 turn by cos/sin[pos, i]; the rest passes.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ d_in, int ld, int q_rank, int kv_off, int rank, int rot, int rdims,
                   const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_len,
                   const int* __restrict__ positions, const int* __restrict__ token_req,
                   const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
                   T* __restrict__ cq, T* __restrict__ pages, int write, int* status) {
  __shared__ float part[8];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const T* row = d_in + (size_t)t * ld;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float x = to_f32(row[i]); sq += x * x; }
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float x = to_f32(row[kv_off + i]); sk += x * x; }
  sq = warp_sum(sq); sk = warp_sum(sk);
  if (lane == 0) { part[warp] = sq; part[4 + warp] = sk; }
  __syncthreads();
  sq = part[0] + part[1] + part[2] + part[3];
  sk = part[4] + part[5] + part[6] + part[7];
  const float iq = 1.0f / sqrtf(sq / (float)q_rank + eps), ik = 1.0f / sqrtf(sk / (float)rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)t * q_rank + i] = from_f32<T>(to_f32(row[i]) * iq * wq[i]);
  if (!write) return;
  if (pos < 0 || (rdims > 0 && pos >= table_len)) {
    if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_BAD_POSITION);
    return;
  }
  const int lp = pos / page_size;
  const int page = lp < max_pages ? block_table[(size_t)token_req[t] * max_pages + lp] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
    return;
  }
  T* dst = pages + ((size_t)page * page_size + (pos % page_size)) * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32(row[kv_off + i]) * ik * wkv[i]);
  const int half = rdims >> 1;
  const T* kr = row + kv_off + rank;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
    const float u = to_f32(kr[2 * i]), v = to_f32(kr[2 * i + 1]);
    dst[rank + 2 * i] = from_f32<T>(u * c - v * s);
    dst[rank + 2 * i + 1] = from_f32<T>(v * c + u * s);
  }
  for (int i = rdims + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = kr[i];
}

KVB_EXPORT int kvb_latent_prep(const void* d_in, int ld, int q_rank, int kv_off, int rank, int rot, int rdims,
                               const float* wq, const float* wkv, float eps, const float* cos_t, const float* sin_t,
                               int table_len, const int* positions, const int* token_req, const int* block_table,
                               int max_pages, int page_size, int num_pages, void* cq, void* pages, int write,
                               int T_, int dtype, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (q_rank < 1 || rank < 1 || rot < 0 || rdims < 0 || (rdims & 1) || rdims > rot) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(latent_prep_kernel<T>, dim3(T_), dim3(128), 0, stream, (const T*)d_in, ld,
                                            q_rank, kv_off, rank, rot, rdims, wq, wkv, eps, cos_t, sin_t, table_len,
                                            positions, token_req, block_table, max_pages, page_size, num_pages,
                                            (T*)cq, (T*)pages, write, status)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- a product per head
// out[t, h * hs_out + n] = sum_k in[t, h * hs_in + k] * W[h, n, k]   for n < N, k < K, h < H.
// Plain FMA in ascending k with float32 sums: an output does not depend on the number of rows.
constexpr int HG_BM = 64, HG_BN = 64, HG_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
head_gemm_kernel(const T* __restrict__ in, int ld_in, int hs_in, const T* __restrict__ W, T* __restrict__ out,
                 int ld_out, int hs_out, int M, int N, int K) {
  __shared__ float As[HG_BK][HG_BM + 4];
  __shared__ float Ws[HG_BK][HG_BN + 4];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.z;
  const T* A = in + (size_t)h * hs_in;
  const T* Wh = W + (size_t)h * N * K;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * HG_BM, n0 = blockIdx.x * HG_BN;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += HG_BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + u][lrow] = (am < M && k < K) ? to_f32(A[(size_t)am * ld_in + k]) : 0.f;
      Ws[lk + u][lrow] = (wn < N && k < K) ? to_f32(Wh[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * ld_out + (size_t)h * hs_out + n] = from_f32<T>(acc[i][j]);
    }
  }
}

KVB_EXPORT int kvb_head_gemm(const void* in, int ld_in, int hs_in, const void* W, void* out, int ld_out, int hs_out,
                             int M, int N, int K, int H, int dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || H <= 0) return 0;
  if (K <= 0 || H > 65535) return KVB_ERR_BAD_SIZE;
  dim3 grid((N + HG_BN - 1) / HG_BN, (M + HG_BM - 1) / HG_BM, H);
  if (grid.y > 65535) return KVB_ERR_BAD_SIZE;
  KVB_DISPATCH_DTYPE(dtype, T, (kvb_launch(head_gemm_kernel<T>, grid, dim3(256), 0, stream, (const T*)in, ld_in, hs_in,
                                            (const T*)W, (T*)out, ld_out, hs_out, M, N, K)));
  return kvb_launch_result();
}

// ---------------------------------------------------------------- attention over the cached rows
// A block takes one query token and up to kLatWarps heads, one head per warp.  The block loads a
// chunk of 32 cached rows into shared memory once for all its heads; a lane scores one key
// (dot over Dc), the warp keeps a running maximum and sum that start from the sink
// (m = sink_h, l = 1: the sink counts once and has no value), and lanes then own value dims.
constexpr int kLatWarps = 8;

template <typename T> struct Word;     // a 4-byte word of shared memory: 1 float or 2 bfloat16
template <> struct Word<float> {
  static constexpr int N = 1;
  static __device__ __forceinline__ float dot(const float* q, unsigned w) { return q[0] * __uint_as_float(w); }
};
template <> struct Word<__nv_bfloat16> {
  static constexpr int N = 2;
  static __device__ __forceinline__ float dot(const float* q, unsigned w) {
    return fmaf(q[1], __uint_as_float(w & 0xffff0000u), q[0] * __uint_as_float(w << 16));
  }
};

template <typename T, int NR>
__global__ void __launch_bounds__(kLatWarps * 32)
latent_attention_kernel(const T* __restrict__ q_abs, int ld_qa, int hs_qa,     // [T, H, rank] absorbed plain part
                        const T* __restrict__ q_raw, int ld_q, int hs_q,        // rotated part before rotation, rot wide
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_len, int rdims,
                        const T* __restrict__ pages, const int* __restrict__ block_table, int max_pages,
                        int page_size, int num_pages, const int* __restrict__ positions,
                        const int* __restrict__ token_req, const float* __restrict__ sink, float scale,
                        T* __restrict__ out, int ld_out, int hs_out, int H, int rank, int rot, int* status) {
  extern __shared__ unsigned lat_smem[];
  constexpr int EW = Word<T>::N;
  const int Dc = rank + rot;
  const int words = Dc / EW;
  const int stride = words | 1;                       // odd: lanes reading one column of a chunk hit 32 banks
  float* q_s = reinterpret_cast<float*>(lat_smem);    // [kLatWarps][Dc]
  unsigned* k_s = lat_smem + kLatWarps * Dc;          // [32][stride]
  __shared__ long long row_of[32];                    // element offset of each key's row, -1: not readable

  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * kLatWarps + warp;
  const bool live = h < H;
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_req[t] * max_pages;
  const bool bad_pos = rdims > 0 && (pos < 0 || pos >= table_len);
  if (bad_pos && threadIdx.x == 0) atomicCAS(status, 0, KVB_STATUS_BAD_POSITION);

  if (live) {
    float* q = q_s + warp * Dc;
    for (int i = lane; i < rank; i += 32) q[i] = to_f32(q_abs[(size_t)t * ld_qa + (size_t)h * hs_qa + i]);
    const T* qr = q_raw + (size_t)t * ld_q + (size_t)h * hs_q;
    const int half = rdims >> 1;
    for (int i = lane; i < half; i += 32) {
      float c = 1.f, s = 0.f;
      if (!bad_pos) { c = cos_t[(size_t)pos * half + i]; s = sin_t[(size_t)pos * half + i]; }
      const float u = to_f32(qr[2 * i]), v = to_f32(qr[2 * i + 1]);
      q[rank + 2 * i] = u * c - v * s;
      q[rank + 2 * i + 1] = v * c + u * s;
    }
    for (int i = rdims + lane; i < rot; i += 32) q[rank + i] = to_f32(qr[i]);
  }
  float m = live ? sink[h] : 0.f, l = 1.f;
  float acc[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) acc[r] = 0.f;

  for (int c0 = 0; c0 <= pos; c0 += 32) {
    const int n_keys = min(32, pos - c0 + 1);
    __syncthreads();                                  // the chunk before is used up (and q_s is written)
    if (threadIdx.x < 32) {
      long long off = -1;
      if (threadIdx.x < n_keys) {
        const int j = c0 + threadIdx.x;
        const int lp = j / page_size;
        const int page = lp < max_pages ? table[lp] : -1;
        if (page < 0 || page >= num_pages) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE);
        else off = ((long long)page * page_size + (j % page_size)) * Dc;
      }
      row_of[threadIdx.x] = off;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_keys * words; idx += blockDim.x) {
      const int j = idx / words, w = idx - j * words;
      const long long off = row_of[j];
      k_s[j * stride + w] = off >= 0 ? reinterpret_cast<const unsigned*>(pages + off)[w] : 0u;
    }
    __syncthreads();
    if (!live) continue;
    const float* q = q_s + warp * Dc;
    float s = -CUDART_INF_F;
    if (lane < n_keys && row_of[lane] >= 0) {
      const unsigned* kr = k_s + lane * stride;
      float dot = 0.f;
      for (int w = 0; w < words; ++w) dot += Word<T>::dot(q + w * EW, kr[w]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float p = s == -CUDART_INF_F ? 0.f : expf(s - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] *= corr;
    const T* kt = reinterpret_cast<const T*>(k_s);
    for (int j = 0; j < n_keys; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const T* vr = kt + (size_t)j * stride * EW;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int i = r * 32 + lane;
        if (i < rank) acc[r] = fmaf(pj, to_f32(vr[i]), acc[r]);
      }
    }
    m = m_new;
  }
  if (!live) return;
  T* o = out + (size_t)t * ld_out + (size_t)h * hs_out;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int i = r * 32 + lane;
    if (i < rank) o[i] = from_f32<T>(acc[r] / l);
  }
}

template <typename T, int NR>
static int launch_latent(const void* q_abs, int ld_qa, int hs_qa, const void* q_raw, int ld_q, int hs_q,
                         const float* cos_t, const float* sin_t, int table_len, int rdims, const void* pages,
                         const int* block_table, int max_pages, int page_size, int num_pages, const int* positions,
                         const int* token_req, const float* sink, float scale, void* out, int ld_out, int hs_out,
                         int T_, int H, int rank, int rot, int* status, cudaStream_t stream) {
  const int Dc = rank + rot;
  const int words = Dc / Word<T>::N;
  const size_t smem = ((size_t)kLatWarps * Dc + 32 * (size_t)(words | 1)) * 4;
  if (smem > 200 * 1024) return KVB_ERR_BAD_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<T, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kvb_launch(latent_attention_kernel<T, NR>, dim3(T_, (H + kLatWarps - 1) / kLatWarps), dim3(kLatWarps * 32), smem,
             stream, (const T*)q_abs, ld_qa, hs_qa, (const T*)q_raw, ld_q, hs_q, cos_t, sin_t, table_len, rdims,
             (const T*)pages, block_table, max_pages, page_size, num_pages, positions, token_req, sink, scale, (T*)out,
             ld_out, hs_out, H, rank, rot, status);
  return kvb_launch_result();
}

// Refuses: rank > 512; in bfloat16 an odd rank + rot or a cache that is not 4-byte aligned.
KVB_EXPORT int kvb_latent_attention(const void* q_abs, int ld_qa, int hs_qa, const void* q_raw, int ld_q, int hs_q,
                                    const float* cos_t, const float* sin_t, int table_len, int rdims,
                                    const void* pages, const int* block_table, int max_pages, int page_size,
                                    int num_pages, const int* positions, const int* token_req, const float* sink,
                                    float scale, void* out, int ld_out, int hs_out, int T_, int H, int rank, int rot,
                                    int dtype, int* status, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (rank < 1 || rank > 512 || rot < 0 || H < 1 || (rdims & 1) || rdims > rot) return KVB_ERR_BAD_SIZE;
  if (dtype == KVB_BF16 && ((rank + rot) & 1)) return KVB_ERR_BAD_SIZE;
  if (reinterpret_cast<uintptr_t>(pages) & 3) return KVB_ERR_ALIGN;
#define KVB_LATENT(NR)                                                                                              \
  KVB_DISPATCH_DTYPE(dtype, T, return (launch_latent<T, NR>(q_abs, ld_qa, hs_qa, q_raw, ld_q, hs_q, cos_t, sin_t,  \
                                                            table_len, rdims, pages, block_table, max_pages,       \
                                                            page_size, num_pages, positions, token_req, sink,      \
                                                            scale, out, ld_out, hs_out, T_, H, rank, rot, status,  \
                                                            stream)))
  if (rank <= 64) { KVB_LATENT(2); }
  else if (rank <= 128) { KVB_LATENT(4); }
  else if (rank <= 256) { KVB_LATENT(8); }
  else { KVB_LATENT(16); }
#undef KVB_LATENT
  return KVB_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------- the same attention on tensor cores (bfloat16)
// A block takes a tile of up to 64 rows, a row being one (token, head) pair: consecutive tokens
// of one request, all heads (at most 64 of them; more heads take further blocks along y).  Keys
// come in chunks of 32 by absolute position.  Per chunk: S = Q K^T by mma.sync m16n8k16 (each of
// the eight warps 16 rows x 16 keys over all of Dc), the scores go through shared memory to a
// softmax step of four threads per row (running maximum and sum start at the sink, as above;
// keys behind a row's own position are masked), the weights come back as bfloat16 and
// O += P V runs on the same chunk in shared memory, whose first `rank` columns are the values
// (each warp 16 rows x half of the value columns, accumulators in registers).  A row's result
// depends on its own query and on the chunks only, not on what else shares its tile.
constexpr int TC_ROWS = 64, TC_KEYS = 32, TC_THREADS = 256, TC_SPAD = 33, TC_PPAD = 40;

__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: tiles of 8 value columns per warp at most (a warp owns half of the value columns): rank <= 16 NT.
template <int NT>
__global__ void __launch_bounds__(TC_THREADS, 1)
latent_attention_tc_kernel(const __nv_bfloat16* __restrict__ q_abs, int ld_qa, int hs_qa,
                           const __nv_bfloat16* __restrict__ q_raw, int ld_q, int hs_q,
                           const float* __restrict__ cos_t, const float* __restrict__ sin_t, int table_len, int rdims,
                           const __nv_bfloat16* __restrict__ pages, const int* __restrict__ block_table, int max_pages,
                           int page_size, int num_pages, const int* __restrict__ positions,
                           const int* __restrict__ q_start, const int* __restrict__ tiles, int tokens_per_tile,
                           const float* __restrict__ sink, float scale, __nv_bfloat16* __restrict__ out, int ld_out,
                           int hs_out, int H, int rank, int rot, int* status) {
  extern __shared__ uint4 tc_smem4[];
  const int Dc = rank + rot, DcP = Dc + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(tc_smem4);              // [64][DcP]
  __nv_bfloat16* Ks0 = Qs + TC_ROWS * DcP;                                      // two buffers of [32][DcP]
  __nv_bfloat16* Ps = Ks0 + 2 * TC_KEYS * DcP;                                  // [64][TC_PPAD]
  float* Ss = reinterpret_cast<float*>(Ps + TC_ROWS * TC_PPAD);                 // [64][TC_SPAD]
  float* m_s = Ss + TC_ROWS * TC_SPAD;
  float* l_s = m_s + TC_ROWS;
  float* corr_s = l_s + TC_ROWS;
  int* pos_s = reinterpret_cast<int*>(corr_s + TC_ROWS);
  __shared__ int row_ok[2][TC_KEYS];              // per buffer: whether the key's row could be read

  pdl_trigger();
  pdl_wait();
  int req, first, ntok;
  if (tiles != nullptr) {
    req = tiles[4 * blockIdx.x]; first = tiles[4 * blockIdx.x + 1]; ntok = tiles[4 * blockIdx.x + 2];
  } else {
    req = blockIdx.x; first = q_start[req]; ntok = q_start[req + 1] - first;
  }
  ntok = min(ntok, tokens_per_tile);
  const int h0 = blockIdx.y * TC_ROWS;
  const int HB = min(TC_ROWS, H - h0);
  const int rows_used = ntok * HB;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* table = block_table + (size_t)req * max_pages;
  const int half = rdims >> 1;

  // the tile's queries: absorbed plain part as it is, the rotated part turned here
  for (int r = warp; r < TC_ROWS; r += TC_THREADS / 32) {
    __nv_bfloat16* q = Qs + (size_t)r * DcP;
    if (r >= rows_used) {
      for (int i = lane; i < DcP; i += 32) q[i] = __float2bfloat16_rn(0.f);
      if (lane == 0) { pos_s[r] = -1; m_s[r] = 0.f; l_s[r] = 1.f; }
      continue;
    }
    const int tl = r / HB, hh = h0 + r - tl * HB;
    const int tr = first + tl;
    const int pos = positions[tr];
    const bool bad_pos = rdims > 0 && (pos < 0 || pos >= table_len);
    if (bad_pos && lane == 0) atomicCAS(status, 0, KVB_STATUS_BAD_POSITION);
    const __nv_bfloat16* qa = q_abs + (size_t)tr * ld_qa + (size_t)hh * hs_qa;
    for (int i = lane; i < rank; i += 32) q[i] = qa[i];
    const __nv_bfloat16* qr = q_raw + (size_t)tr * ld_q + (size_t)hh * hs_q;
    for (int i = lane; i < half; i += 32) {
      float c = 1.f, sn = 0.f;
      if (!bad_pos) { c = cos_t[(size_t)pos * half + i]; sn = sin_t[(size_t)pos * half + i]; }
      const float u = __bfloat162float(qr[2 * i]), v = __bfloat162float(qr[2 * i + 1]);
      q[rank + 2 * i] = __float2bfloat16_rn(u * c - v * sn);
      q[rank + 2 * i + 1] = __float2bfloat16_rn(v * c + u * sn);
    }
    for (int i = rdims + lane; i < rot; i += 32) q[rank + i] = qr[i];
    for (int i = Dc + lane; i < DcP; i += 32) q[i] = __float2bfloat16_rn(0.f);
    if (lane == 0) { pos_s[r] = pos; m_s[r] = sink[hh]; l_s[r] = 1.f; }
  }
  const int max_pos = ntok > 0 ? positions[first + ntok - 1] : -1;

  const int g = lane >> 2, t4 = lane & 3;
  const int mrow = (warp & 3) * 16;
  const int nt_used = rank / 16;                 // tiles of 8 columns in this warp's half of the values
  const int ncol0 = (warp >> 2) * (rank / 2);
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }

  // A chunk's rows are requested (cp.async, 16 bytes a piece) one chunk ahead, into the other buffer.
  const int vecs = Dc >> 3;                        // 16-byte pieces per row
  auto request_chunk = [&](int c0, int buf) {
    __nv_bfloat16* Kb = Ks0 + (size_t)buf * TC_KEYS * DcP;
    for (int j = warp; j < TC_KEYS; j += TC_THREADS / 32) {
      const int key = c0 + j;
      long long off = -1;
      if (key <= max_pos) {
        const int lp = key / page_size;
        const int page = lp < max_pages ? table[lp] : -1;
        if (page < 0 || page >= num_pages) { if (lane == 0) atomicCAS(status, 0, KVB_STATUS_UNMAPPED_PAGE); }
        else off = ((long long)page * page_size + (key % page_size)) * Dc;
      }
      if (lane == 0) row_ok[buf][j] = off >= 0;
      __nv_bfloat16* dst = Kb + (size_t)j * DcP;
      if (off >= 0) {
        const __nv_bfloat16* src = pages + off;
        for (int v = lane; v < vecs; v += 32) {
          const unsigned d = (unsigned)__cvta_generic_to_shared(dst + 8 * v);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(d), "l"(src + 8 * v) : "memory");
        }
      } else {
        for (int v = lane; v < vecs; v += 32) reinterpret_cast<uint4*>(dst)[v] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (max_pos >= 0) request_chunk(0, 0);
  const bool row_group_live = mrow < rows_used;   // a warp whose 16 rows are all empty only keeps the barriers
  int it = 0;
  for (int c0 = 0; c0 <= max_pos; c0 += TC_KEYS, ++it) {
    const int n_keys = min(TC_KEYS, max_pos - c0 + 1);
    const __nv_bfloat16* Ks = Ks0 + (size_t)(it & 1) * TC_KEYS * DcP;
    const int* ok = row_ok[it & 1];
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                               // this chunk has arrived; the chunk before is used up (first round: Qs and the row state are written)
    if (c0 + TC_KEYS <= max_pos) request_chunk(c0 + TC_KEYS, (it + 1) & 1);
    // ---- scores: this warp's 16 rows against 16 of the chunk's keys
    if (row_group_live) {
      const int kcol = (warp >> 2) * 16;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      const __nv_bfloat16* a_ptr = Qs + (size_t)(mrow + (lane & 15)) * DcP + (lane >> 4) * 8;
      const __nv_bfloat16* b_ptr = Ks + (size_t)(kcol + ((lane >> 4) << 3) + (lane & 7)) * DcP + ((lane >> 3) & 1) * 8;
      // two sets of sums, for the even and the odd steps along Dc: four chains of dependent products instead
      // of two, and the operands of a pair of steps are fetched together (the same order for every row)
      float u0[4] = {0.f, 0.f, 0.f, 0.f}, u1[4] = {0.f, 0.f, 0.f, 0.f};
      int ks = 0;
      for (; ks + 32 <= Dc; ks += 32) {
        unsigned a0, a1, a2, a3, b0, b1, b2, b3, c0_, c1_, c2_, c3_, d0, d1, d2, d3;
        ldsm_x4(a0, a1, a2, a3, a_ptr + ks);
        ldsm_x4(b0, b1, b2, b3, b_ptr + ks);
        ldsm_x4(c0_, c1_, c2_, c3_, a_ptr + ks + 16);
        ldsm_x4(d0, d1, d2, d3, b_ptr + ks + 16);
        mma_bf16_16816(s0, a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s1, a0, a1, a2, a3, b2, b3);
        mma_bf16_16816(u0, c0_, c1_, c2_, c3_, d0, d1);
        mma_bf16_16816(u1, c0_, c1_, c2_, c3_, d2, d3);
      }
      if (ks < Dc) {
        unsigned a0, a1, a2, a3, b0, b1, b2, b3;
        ldsm_x4(a0, a1, a2, a3, a_ptr + ks);
        ldsm_x4(b0, b1, b2, b3, b_ptr + ks);
        mma_bf16_16816(s0, a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(s1, a0, a1, a2, a3, b2, b3);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) { s0[e] += u0[e]; s1[e] += u1[e]; }
      float* srow = Ss + (size_t)(mrow + g) * TC_SPAD + kcol + 2 * t4;
      srow[0] = s0[0] * scale; srow[1] = s0[1] * scale; srow[8] = s1[0] * scale; srow[9] = s1[1] * scale;
      srow += 8 * TC_SPAD;
      srow[0] = s0[2] * scale; srow[1] = s0[3] * scale; srow[8] = s1[2] * scale; srow[9] = s1[3] * scale;
    }
    __syncthreads();
    // ---- softmax step: four threads per row, eight keys each
    {
      const int row = tid >> 2, k0 = (tid & 3) * 8;
      const int pos_r = pos_s[row];
      float sv[8], mx = -CUDART_INF_F;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int kk = k0 + e;
        const bool valid = kk < n_keys && c0 + kk <= pos_r && ok[kk];
        sv[e] = valid ? Ss[(size_t)row * TC_SPAD + kk] : -CUDART_INF_F;
        mx = fmaxf(mx, sv[e]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_old = m_s[row];
      const float m_new = fmaxf(m_old, mx);
      float psum = 0.f;
      __nv_bfloat16* prow = Ps + (size_t)row * TC_PPAD + k0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float p = sv[e] == -CUDART_INF_F ? 0.f : expf(sv[e] - m_new);
        psum += p;
        prow[e] = __float2bfloat16_rn(p);
      }
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      psum += __shfl_xor_sync(0xffffffffu, psum, 2);
      if ((tid & 3) == 0) {
        const float corr = expf(m_old - m_new);
        m_s[row] = m_new;
        l_s[row] = l_s[row] * corr + psum;
        corr_s[row] = corr;
      }
    }
    __syncthreads();
    // ---- O = O * corr + P V for this warp's 16 rows and its half of the value columns
    if (row_group_live) {
      const float c_lo = corr_s[mrow + g], c_hi = corr_s[mrow + g + 8];
#pragma unroll
      for (int n = 0; n < NT; ++n) { acc[n][0] *= c_lo; acc[n][1] *= c_lo; acc[n][2] *= c_hi; acc[n][3] *= c_hi; }
      const __nv_bfloat16* a_ptr = Ps + (size_t)(mrow + (lane & 15)) * TC_PPAD + (lane >> 4) * 8;
      const __nv_bfloat16* b_ptr = Ks + (size_t)(((lane >> 3) & 1) * 8 + (lane & 7)) * DcP + ncol0 + (lane >> 4) * 8;
#pragma unroll
      for (int ks = 0; ks < TC_KEYS; ks += 16) {
        unsigned a0, a1, a2, a3;
        ldsm_x4(a0, a1, a2, a3, a_ptr + ks);
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          if (2 * np < nt_used) {
            unsigned b0, b1, b2, b3;
            ldsm_x4_trans(b0, b1, b2, b3, b_ptr + (size_t)ks * DcP + np * 16);
            mma_bf16_16816(acc[2 * np], a0, a1, a2, a3, b0, b1);
            mma_bf16_16816(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int hrow = 0; hrow < 2; ++hrow) {
    const int r = mrow + g + 8 * hrow;
    if (r >= rows_used) continue;
    const int tl = r / HB, hh = h0 + r - tl * HB;
    const float inv = 1.0f / l_s[r];
    __nv_bfloat16* o = out + (size_t)(first + tl) * ld_out + (size_t)hh * hs_out + ncol0 + 2 * t4;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      if (n < nt_used) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(acc[n][2 * hrow] * inv, acc[n][2 * hrow + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(o + n * 8) = v;
      }
    }
  }
}

// Rows of (token, head) pairs per tile: tokens per tile for a number of heads.
KVB_EXPORT int kvb_latent_attention_tc_tokens_per_tile(int H) { return H >= TC_ROWS ? 1 : TC_ROWS / H; }

// Whether the tensor-core form takes these sizes: rank a multiple of 32 up to 512, rank + rot a multiple of 16.
KVB_EXPORT int kvb_latent_attention_tc_supported(int rank, int rot) {
  return rank >= 32 && rank <= 512 && rank % 32 == 0 && (rank + rot) % 16 == 0 ? 1 : 0;
}

template <int NT>
static int launch_latent_tc(const void* q_abs, int ld_qa, int hs_qa, const void* q_raw, int ld_q, int hs_q,
                            const float* cos_t, const float* sin_t, int table_len, int rdims, const void* pages,
                            const int* block_table, int max_pages, int page_size, int num_pages, const int* positions,
                            const int* q_start, const int* tiles, int n_tiles, const float* sink, float scale, void* out,
                            int ld_out, int hs_out, int H, int rank, int rot, int* status, cudaStream_t stream) {
  const int DcP = rank + rot + 8;
  const size_t smem = (size_t)(TC_ROWS + 2 * TC_KEYS) * DcP * 2 + (size_t)TC_ROWS * TC_PPAD * 2 +
                      (size_t)TC_ROWS * TC_SPAD * 4 + 4 * TC_ROWS * 4;
  if (smem > 220 * 1024) return KVB_ERR_BAD_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_tc_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  using B = __nv_bfloat16;
  kvb_launch(latent_attention_tc_kernel<NT>, dim3(n_tiles, (H + TC_ROWS - 1) / TC_ROWS), dim3(TC_THREADS), smem, stream,
             (const B*)q_abs, ld_qa, hs_qa, (const B*)q_raw, ld_q, hs_q, cos_t, sin_t, table_len, rdims, (const B*)pages,
             block_table, max_pages, page_size, num_pages, positions, q_start, tiles,
             kvb_latent_attention_tc_tokens_per_tile(H), sink, scale, (B*)out, ld_out, hs_out, H, rank, rot, status);
  return kvb_launch_result();
}

// tiles: [n_tiles, 4] int32 rows (request row, first token row, tokens, 0) of at most
// kvb_latent_attention_tc_tokens_per_tile(H) tokens each, or null: one tile per request (n_tiles requests, each
// bringing at most that many tokens).  Everything 16-byte aligned: the cache, and rows of rank + rot elements.
KVB_EXPORT int kvb_latent_attention_tc(const void* q_abs, int ld_qa, int hs_qa, const void* q_raw, int ld_q, int hs_q,
                                       const float* cos_t, const float* sin_t, int table_len, int rdims,
                                       const void* pages, const int* block_table, int max_pages, int page_size,
                                       int num_pages, const int* positions, const int* q_start, const int* tiles,
                                       int n_tiles, const float* sink, float scale, void* out, int ld_out, int hs_out,
                                       int H, int rank, int rot, int* status, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!kvb_latent_attention_tc_supported(rank, rot) || H < 1 || (rdims & 1) || rdims > rot) return KVB_ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(pages) & 15) || (reinterpret_cast<uintptr_t>(out) & 3) || (ld_out & 1) || (hs_out & 1))
    return KVB_ERR_ALIGN;
#define KVB_LATENT_TC(NT)                                                                                            \
  return launch_latent_tc<NT>(q_abs, ld_qa, hs_qa, q_raw, ld_q, hs_q, cos_t, sin_t, table_len, rdims, pages,        \
                              block_table, max_pages, page_size, num_pages, positions, q_start, tiles, n_tiles, sink, \
                              scale, out, ld_out, hs_out, H, rank, rot, status, stream)
  if (rank <= 64) { KVB_LATENT_TC(4); }
  if (rank <= 128) { KVB_LATENT_TC(8); }
  if (rank <= 256) { KVB_LATENT_TC(16); }
  KVB_LATENT_TC(32);
#undef KVB_LATENT_TC
}
