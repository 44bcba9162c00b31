// latent_attn.cu — attention over a paged cache of compressed key/value latents.
//
// Every cached token is one row [c (rank) | kr (rd)]: the normalised latent c, from which each
// head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c), and one rotary key part kr
// shared by all heads.  With the key map folded into the query (qa_h = Uk_h^T q_h) a head's score is
//     s = (qa_h . c + qr_h . kr) * scale
// and its output is Uv_h (sum_j p_j c_j): the kernel works entirely in the latent space, as
// multi-query attention with key width rank + rd and value width rank.
//
//   latent_prepare : per token  c = rmsnorm(dkv[:rank]) * w -> cache ; kr = rope(dkv[rank:]) -> cache ;
//                    rope on the rotary part of every query head in place.  Angles pos * f_i, cos
//                    and sin in fp32; pairs are interleaved (2i, 2i+1); `mult` scales cos and sin.
//   latent_attn    : causal softmax attention of packed query rows over the paged rows; scores,
//                    weights and accumulators in fp32.  One CTA per (token, group of 8 heads), one
//                    warp per head, 32-key tiles staged once per CTA in shared memory.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kHeadsPerCta = 8;
constexpr int kTileKeys = 32;

template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ q, int64_t ldq, const T* __restrict__ dkv,
                                      int64_t ld_dkv, T* __restrict__ cache, int64_t ldc,
                                      const float* __restrict__ cw, const float* __restrict__ inv_freq,
                                      float mult, const int* __restrict__ positions,
                                      const int* __restrict__ slots, int H, int dim, int rd, int dims,
                                      int rank, float eps) {
  extern __shared__ float cs[];  // [dims / 2] cos, [dims / 2] sin
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int np = dims / 2;
  const float pos = (float)positions[row];
  const T* src = dkv + (size_t)row * ld_dkv;
  T* dst = cache + (size_t)slots[row] * ldc;
  for (int i = threadIdx.x; i < np; i += blockDim.x) {
    const float a = pos * inv_freq[i];
    cs[i] = cosf(a) * mult;
    cs[np + i] = sinf(a) * mult;
  }
  float ss = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = Num<T>::to_f(src[i]);
    ss += v * v;
  }
  ss = block_sum<128>(ss, red);   // also orders the cos / sin table before its readers
  const float r = rsqrtf(ss / (float)rank + eps);
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    dst[i] = Num<T>::from_f(Num<T>::to_f(src[i]) * r * cw[i]);
  for (int i = threadIdx.x; i < rd - dims; i += blockDim.x) dst[rank + dims + i] = src[rank + dims + i];
  const int tasks = (H + 1) * np;
  for (int k = threadIdx.x; k < tasks; k += blockDim.x) {
    const int hh = k / np, i = k - hh * np;
    const float c = cs[i], s = cs[np + i];
    if (hh < H) {
      T* p = q + (size_t)row * ldq + (size_t)hh * (dim + rd) + dim + 2 * i;
      const float u = Num<T>::to_f(p[0]), v = Num<T>::to_f(p[1]);
      p[0] = Num<T>::from_f(u * c - v * s);
      p[1] = Num<T>::from_f(v * c + u * s);
    } else {
      const float u = Num<T>::to_f(src[rank + 2 * i]), v = Num<T>::to_f(src[rank + 2 * i + 1]);
      dst[rank + 2 * i] = Num<T>::from_f(u * c - v * s);
      dst[rank + 2 * i + 1] = Num<T>::from_f(v * c + u * s);
    }
  }
}

template <typename T, typename QA, int NR>
__global__ void __launch_bounds__(kHeadsPerCta * 32)
latent_attn_kernel(T* __restrict__ out, int64_t out_hs, int64_t out_ts, const QA* __restrict__ qa,
                   int64_t qa_hs, int64_t qa_ts, const T* __restrict__ q, int64_t ldq,
                   const T* __restrict__ cache, int64_t ldc, const int* __restrict__ q_cu,
                   const int* __restrict__ kv_cu, const int* __restrict__ tables,
                   const int* __restrict__ blk_cu, const int* __restrict__ token_seq, int H, int dim,
                   int rd, int rank, int block_size, float scale) {
  extern __shared__ float sm[];
  const int Dk = rank + rd, ldk = Dk + 1;
  float* qs = sm;                           // [kHeadsPerCta][Dk]
  float* Ks = sm + kHeadsPerCta * Dk;       // [kTileKeys][ldk]
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * kHeadsPerCta + warp;
  const int seq = token_seq[row];
  const int q_len = q_cu[seq + 1] - q_cu[seq], kv_len = kv_cu[seq + 1] - kv_cu[seq];
  const int pos = kv_len - q_len + (row - q_cu[seq]);   // last visible key
  const int* table = tables + blk_cu[seq];
  if (h < H) {
    const QA* a = qa + (size_t)h * qa_hs + (size_t)row * qa_ts;
    for (int d = lane; d < rank; d += 32) qs[warp * Dk + d] = Num<QA>::to_f(a[d]);
    const T* r = q + (size_t)row * ldq + (size_t)h * (dim + rd) + dim;
    for (int d = lane; d < rd; d += 32) qs[warp * Dk + rank + d] = Num<T>::to_f(r[d]);
  }
  float acc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) acc[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;
  for (int j0 = 0; j0 <= pos; j0 += kTileKeys) {
    __syncthreads();   // previous tile fully consumed (and qs written, first time round)
    for (int jj = warp; jj < kTileKeys; jj += kHeadsPerCta) {
      const int key = j0 + jj;
      float* dstk = Ks + jj * ldk;
      if (key <= pos) {
        const T* srck = cache + ((size_t)table[key / block_size] + key % block_size) * ldc;
        for (int d = lane; d < Dk; d += 32) dstk[d] = Num<T>::to_f(srck[d]);
      } else {
        for (int d = lane; d < Dk; d += 32) dstk[d] = 0.0f;
      }
    }
    __syncthreads();
    if (h < H) {
      const float* qh = qs + warp * Dk;
      const float* kj = Ks + lane * ldk;
      float s = 0.0f;
      for (int d = 0; d < Dk; ++d) s += qh[d] * kj[d];
      s = (j0 + lane <= pos) ? s * scale : -INFINITY;
      float mx = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m, mx);
      const float p = expf(s - m_new);
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < NR; ++i) acc[i] *= corr;
      for (int jj = 0; jj < kTileKeys; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const float* kr = Ks + jj * ldk;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int r = lane + 32 * i;
          if (r < rank) acc[i] += pj * kr[r];
        }
      }
    }
  }
  if (h < H) {
    const float inv = 1.0f / l;
    T* o = out + (size_t)h * out_hs + (size_t)row * out_ts;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int r = lane + 32 * i;
      if (r < rank) o[r] = Num<T>::from_f(acc[i] * inv);
    }
  }
}

template <typename T, typename QA, int NR>
int launch_latent_attn(void* out, int64_t out_hs, int64_t out_ts, const void* qa, int64_t qa_hs,
                       int64_t qa_ts, const void* q, int64_t ldq, const void* cache, int64_t ldc,
                       const int* q_cu, const int* kv_cu, const int* tables, const int* blk_cu,
                       const int* token_seq, int64_t rows, int H, int dim, int rd, int rank,
                       int block_size, float scale, cudaStream_t st) {
  const int Dk = rank + rd;
  const size_t smem = ((size_t)kHeadsPerCta * Dk + (size_t)kTileKeys * (Dk + 1)) * sizeof(float);
  B200_CHECK_ARG(smem <= 200 * 1024, "latent_attn: rank + rot_dim = %d does not fit in shared memory", Dk);
  auto kern = latent_attn_kernel<T, QA, NR>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)rows, (unsigned)((H + kHeadsPerCta - 1) / kHeadsPerCta));
  kern<<<grid, kHeadsPerCta * 32, smem, st>>>(static_cast<T*>(out), out_hs, out_ts,
                                              static_cast<const QA*>(qa), qa_hs, qa_ts,
                                              static_cast<const T*>(q), ldq, static_cast<const T*>(cache),
                                              ldc, q_cu, kv_cu, tables, blk_cu, token_seq, H, dim, rd, rank,
                                              block_size, scale);
  B200_LAUNCH_OK("latent_attn_kernel");
  return B200_OK;
}

template <typename T, typename QA>
int dispatch_nr(int rank, void* out, int64_t out_hs, int64_t out_ts, const void* qa, int64_t qa_hs,
                int64_t qa_ts, const void* q, int64_t ldq, const void* cache, int64_t ldc, const int* q_cu,
                const int* kv_cu, const int* tables, const int* blk_cu, const int* token_seq, int64_t rows,
                int H, int dim, int rd, int block_size, float scale, cudaStream_t st) {
#define LA_ARGS out, out_hs, out_ts, qa, qa_hs, qa_ts, q, ldq, cache, ldc, q_cu, kv_cu, tables, blk_cu, \
                token_seq, rows, H, dim, rd, rank, block_size, scale, st
  const int nr = (rank + 31) / 32;
  if (nr <= 2) return launch_latent_attn<T, QA, 2>(LA_ARGS);
  if (nr <= 4) return launch_latent_attn<T, QA, 4>(LA_ARGS);
  if (nr <= 8) return launch_latent_attn<T, QA, 8>(LA_ARGS);
  if (nr <= 16) return launch_latent_attn<T, QA, 16>(LA_ARGS);
#undef LA_ARGS
  return set_error(B200_ERR_UNSUPPORTED, "latent_attn: latent rank %d > 512", rank);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_latent_prepare(void* q, int64_t ldq, const void* dkv, int64_t ld_dkv, void* cache, int64_t ldc,
                        const float* c_norm_weight, const float* inv_freq, float mult,
                        const int32_t* positions, const int32_t* slots, int64_t rows, int64_t H,
                        int64_t dim, int64_t rd, int64_t dims, int64_t rank, float eps, int dtype,
                        b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(q && dkv && cache && c_norm_weight && inv_freq && positions && slots,
                 "latent_prepare: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && dim >= 0 && rd >= 0 && rank > 0 && dims >= 0 && dims <= rd &&
                     dims % 2 == 0 && dims <= 4096 && ldq >= H * (dim + rd) && ld_dkv >= rank + rd &&
                     ldc >= rank + rd,
                 "latent_prepare: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)dims * sizeof(float);
#define LP_LAUNCH(T)                                                                                   \
  latent_prepare_kernel<T><<<(unsigned)rows, 128, smem, st>>>(                                          \
      static_cast<T*>(q), ldq, static_cast<const T*>(dkv), ld_dkv, static_cast<T*>(cache), ldc,          \
      c_norm_weight, inv_freq, mult, positions, slots, (int)H, (int)dim, (int)rd, (int)dims, (int)rank, eps)
  switch (dtype) {
    case B200_BF16: LP_LAUNCH(__nv_bfloat16); break;
    case B200_FP16: LP_LAUNCH(__half); break;
    case B200_FP32: LP_LAUNCH(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef LP_LAUNCH
  B200_LAUNCH_OK("latent_prepare_kernel");
  return B200_OK;
}

int b200_latent_attn(void* out, int64_t out_head_stride, int64_t out_token_stride, const void* q_absorbed,
                     int64_t qa_head_stride, int64_t qa_token_stride, int qa_is_fp32, const void* q,
                     int64_t ldq, const void* cache, int64_t ldc, const int32_t* q_cu_lens,
                     const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                     const int32_t* token_seq, int64_t rows, int64_t H, int64_t dim, int64_t rd,
                     int64_t rank, int64_t block_size, float scale, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && q_absorbed && q && cache && q_cu_lens && kv_cu_lens && block_tables &&
                     cu_block_lens && token_seq,
                 "latent_attn: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && H <= 65535 * kHeadsPerCta && dim >= 0 && rd >= 0 && rank > 0 &&
                     block_size > 0 && ldq >= H * (dim + rd) && ldc >= rank + rd,
                 "latent_attn: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
#define LA_CALL(T, QA)                                                                                  \
  return dispatch_nr<T, QA>((int)rank, out, out_head_stride, out_token_stride, q_absorbed, qa_head_stride, \
                            qa_token_stride, q, ldq, cache, ldc, q_cu_lens, kv_cu_lens, block_tables,    \
                            cu_block_lens, token_seq, rows, (int)H, (int)dim, (int)rd, (int)block_size,   \
                            scale, st)
  switch (dtype) {
    case B200_BF16:
      if (qa_is_fp32) { LA_CALL(__nv_bfloat16, float); }
      LA_CALL(__nv_bfloat16, __nv_bfloat16);
    case B200_FP32:
      LA_CALL(float, float);
    default:
      return set_error(B200_ERR_UNSUPPORTED, "latent_attn: bf16 or fp32 activations");
  }
#undef LA_CALL
}

}  // extern "C"
