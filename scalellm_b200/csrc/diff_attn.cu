// diff_attn.cu — differential attention over a paged cache with a sliding window that keeps a
// sequence's first tokens.
//
// Every head carries TWO query/key maps of width `dim` over ONE set of values of width `vdim`:
//     s1_j = scale * q1 . k1_j ,  s2_j = scale * q2 . k2_j            over the visible keys j
//     a1 = softmax(s1) V ,  a2 = softmax(s2) V
//     o  = a1 - lambda a2 ;  o <- o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)
// Key j is visible from position i when j <= i and (i - j < window or j < keep_first).  Query head h reads
// key/value head h / (H / G).  Queries and keys are RMS-normalised per head and map (weight shared by all heads
// and maps) and then rotated: pairs (2i, 2i + 1) of the first `rot_dims` channels of every map turn by
// position * inv_freq[i], with cos and sin multiplied by `rot_mult`.
//
//   prepare : q rows -> fp32 [rows, H, 2, dim]; k rows -> K cache [slots, G, 2 * dim]; v rows -> V cache
//             [slots, G, vdim] (cache entries have the activation type T)
//   attend  : one CTA per (row, head); every warp walks its share of the visible keys in groups of 32 (lane =
//             key for the two scores, lane = value channel for the weighted sum) with a running maximum and sum
//             per map; the warps' partial results are merged through shared memory.
// Scores, softmax weights, sums, the norm and the gate are fp32.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarps = 4;
constexpr int kMaxVPerLane = 8;      // vdim <= 256

template <typename T>
__device__ __forceinline__ void norm_rotate_unit(const T* __restrict__ src, const float* __restrict__ w,
                                                 const float* __restrict__ inv_freq, float rot_mult, int rot_dims,
                                                 int dim, float eps, float pos, int lane, float* dst32,
                                                 T* dstT) {
  float ss = 0.0f;
  for (int i = lane; i < dim; i += 32) {
    const float v = Num<T>::to_f(src[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)dim + eps);
  const int pairs = (dim + 1) / 2;
  for (int p = lane; p < pairs; p += 32) {
    const int i0 = 2 * p, i1 = 2 * p + 1;
    float a = Num<T>::to_f(src[i0]) * r * w[i0];
    float b = i1 < dim ? Num<T>::to_f(src[i1]) * r * w[i1] : 0.0f;
    if (i1 < rot_dims) {
      const float ang = pos * inv_freq[p];
      const float c = cosf(ang) * rot_mult, s = sinf(ang) * rot_mult;
      const float ra = a * c - b * s, rb = b * c + a * s;
      a = ra;
      b = rb;
    }
    if (dst32) {
      dst32[i0] = a;
      if (i1 < dim) dst32[i1] = b;
    } else {
      dstT[i0] = Num<T>::from_f(a);
      if (i1 < dim) dstT[i1] = Num<T>::from_f(b);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
diff_attn_prepare_kernel(float* __restrict__ q_out, const T* __restrict__ q_in, const T* __restrict__ k_in,
                         const T* __restrict__ v_in, int64_t ld, T* __restrict__ k_cache, T* __restrict__ v_cache,
                         const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                         const float* __restrict__ inv_freq, float rot_mult, const int* __restrict__ positions,
                         const int* __restrict__ slots, int H, int G, int dim, int vdim, int rot_dims, float eps) {
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float pos = (float)positions[row];
  const int n_q = H * 2, n_k = k_in ? G * 2 : 0;
  const size_t slot = k_in ? (size_t)slots[row] : 0;
  for (int u = warp; u < n_q + n_k; u += kWarps) {
    if (u < n_q) {
      norm_rotate_unit<T>(q_in + (size_t)row * ld + (size_t)u * dim, q_norm_w, inv_freq, rot_mult, rot_dims, dim,
                          eps, pos, lane, q_out + ((size_t)row * n_q + u) * dim, nullptr);
    } else {
      const int uk = u - n_q;
      norm_rotate_unit<T>(k_in + (size_t)row * ld + (size_t)uk * dim, k_norm_w, inv_freq, rot_mult, rot_dims, dim,
                          eps, pos, lane, nullptr, k_cache + (slot * n_k + uk) * dim);
    }
  }
  if (v_in) {
    const int nv = G * vdim;
    for (int i = threadIdx.x; i < nv; i += kWarps * 32) v_cache[slot * nv + i] = v_in[(size_t)row * ld + i];
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
diff_attn_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ q, const T* __restrict__ k_cache,
                 const T* __restrict__ v_cache, const T* __restrict__ gate, int64_t ldg,
                 const int* __restrict__ q_cu, const int* __restrict__ kv_cu, const int* __restrict__ block_tables,
                 const int* __restrict__ cu_block_lens, const int* __restrict__ token_seq, int H, int G, int dim,
                 int vdim, int block_size, float scale, int window, int keep_first, float lambda, float out_scale,
                 float eps) {
  extern __shared__ float sm[];
  float* q_s = sm;                                   // [2 * dim]
  float* acc_s = q_s + 2 * dim;                      // [kWarps][2][vdim]
  float* ml_s = acc_s + kWarps * 2 * vdim;           // [kWarps][4]  m1 l1 m2 l2
  __shared__ float red[32];
  const int row = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = token_seq[row];
  const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
  const int i = kv_len - q_len + (row - q_cu[seq]);            // position of this row
  const int g = h / (H / G);
  const int* table = block_tables + cu_block_lens[seq];
  for (int d = threadIdx.x; d < 2 * dim; d += kWarps * 32) q_s[d] = q[((size_t)row * H + h) * 2 * dim + d];
  __syncthreads();
  // visible keys: the kept first tokens that have left the window, then the window
  const int lo = (window > 0 && i - window + 1 > 0) ? i - window + 1 : 0;
  const int ns = keep_first < lo ? keep_first : lo;
  const int total = ns + (i - lo + 1);
  const size_t k_stride = (size_t)G * 2 * dim, v_stride = (size_t)G * vdim;
  float m1 = -INFINITY, l1 = 0.0f, m2 = -INFINITY, l2 = 0.0f;
  float a1[kMaxVPerLane], a2[kMaxVPerLane];
#pragma unroll
  for (int c = 0; c < kMaxVPerLane; ++c) a1[c] = a2[c] = 0.0f;
  for (int n0 = warp * 32; n0 < total; n0 += kWarps * 32) {
    const int n = n0 + lane;
    const bool live = n < total;
    int slot = 0;
    float s1 = -INFINITY, s2 = -INFINITY;
    if (live) {
      const int j = n < ns ? n : lo + (n - ns);
      slot = table[j / block_size] + j % block_size;
      const T* kr = k_cache + (size_t)slot * k_stride + (size_t)g * 2 * dim;
      float d1 = 0.0f, d2 = 0.0f;
      for (int d = 0; d < dim; ++d) {
        d1 += q_s[d] * Num<T>::to_f(kr[d]);
        d2 += q_s[dim + d] * Num<T>::to_f(kr[dim + d]);
      }
      s1 = d1 * scale;
      s2 = d2 * scale;
    }
    float t1 = s1, t2 = s2;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, o));
      t2 = fmaxf(t2, __shfl_xor_sync(0xffffffffu, t2, o));
    }
    const float nm1 = fmaxf(m1, t1), nm2 = fmaxf(m2, t2);     // finite: lane 0 of a started group is live
    const float c1 = expf(m1 - nm1), c2 = expf(m2 - nm2);
    const float p1 = live ? expf(s1 - nm1) : 0.0f, p2 = live ? expf(s2 - nm2) : 0.0f;
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
    m1 = nm1;
    m2 = nm2;
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) { a1[c] *= c1; a2[c] *= c2; }
    const int cnt = total - n0 < 32 ? total - n0 : 32;
    for (int kk = 0; kk < cnt; ++kk) {
      const float w1 = __shfl_sync(0xffffffffu, p1, kk), w2 = __shfl_sync(0xffffffffu, p2, kk);
      const int sl = __shfl_sync(0xffffffffu, slot, kk);
      const T* vr = v_cache + (size_t)sl * v_stride + (size_t)g * vdim;
#pragma unroll
      for (int c = 0; c < kMaxVPerLane; ++c) {
        const int col = lane + 32 * c;
        if (col < vdim) {
          const float v = Num<T>::to_f(vr[col]);
          a1[c] += w1 * v;
          a2[c] += w2 * v;
        }
      }
    }
  }
  // merge the warps
  if (lane == 0) {
    ml_s[warp * 4 + 0] = m1; ml_s[warp * 4 + 1] = l1; ml_s[warp * 4 + 2] = m2; ml_s[warp * 4 + 3] = l2;
  }
#pragma unroll
  for (int c = 0; c < kMaxVPerLane; ++c) {
    const int col = lane + 32 * c;
    if (col < vdim) {
      acc_s[(warp * 2 + 0) * vdim + col] = a1[c];
      acc_s[(warp * 2 + 1) * vdim + col] = a2[c];
    }
  }
  __syncthreads();
  float M1 = -INFINITY, M2 = -INFINITY;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) { M1 = fmaxf(M1, ml_s[w * 4]); M2 = fmaxf(M2, ml_s[w * 4 + 2]); }
  float L1 = 0.0f, L2 = 0.0f, f1[kWarps], f2[kWarps];
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    f1[w] = ml_s[w * 4 + 1] > 0.0f ? expf(ml_s[w * 4] - M1) : 0.0f;
    f2[w] = ml_s[w * 4 + 3] > 0.0f ? expf(ml_s[w * 4 + 2] - M2) : 0.0f;
    L1 += f1[w] * ml_s[w * 4 + 1];
    L2 += f2[w] * ml_s[w * 4 + 3];
  }
  float o[2] = {0.0f, 0.0f};       // up to two value channels per thread (vdim <= 256, 128 threads)
  float ss = 0.0f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int col = threadIdx.x + r * kWarps * 32;
    if (col < vdim) {
      float x1 = 0.0f, x2 = 0.0f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        x1 += f1[w] * acc_s[(w * 2 + 0) * vdim + col];
        x2 += f2[w] * acc_s[(w * 2 + 1) * vdim + col];
      }
      o[r] = x1 / L1 - lambda * (x2 / L2);
      ss += o[r] * o[r];
    }
  }
  ss = block_sum<kWarps * 32>(ss, red);
  const float gl = gate ? 1.0f / (1.0f + expf(-Num<T>::to_f(gate[(size_t)row * ldg + h]))) : 1.0f;
  const float f = out_scale * gl / sqrtf(ss / (float)vdim + eps);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int col = threadIdx.x + r * kWarps * 32;
    if (col < vdim) out[(size_t)row * ldo + (size_t)h * vdim + col] = Num<T>::from_f(o[r] * f);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_diff_attn_prepare(float* q_out, const void* q_in, const void* k_in, const void* v_in, int64_t ld,
                           void* k_cache, void* v_cache, const float* q_norm_weight, const float* k_norm_weight,
                           const float* inv_freq, float rot_mult, const int32_t* positions, const int32_t* slots,
                           int64_t rows, int64_t H, int64_t G, int64_t dim, int64_t vdim, int64_t rot_dims,
                           float eps, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(q_out && q_in && q_norm_weight && positions, "diff_attn_prepare: null pointer");
  B200_CHECK_ARG(!k_in || (v_in && k_cache && v_cache && k_norm_weight && slots),
                 "diff_attn_prepare: keys without values, caches, norm weight or slots");
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && rot_dims >= 0 &&
                     rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq) && ld >= H * 2 * dim,
                 "diff_attn_prepare: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
#define DP_CALL(T)                                                                                             \
  diff_attn_prepare_kernel<T><<<(unsigned)rows, kWarps * 32, 0, st>>>(                                         \
      q_out, static_cast<const T*>(q_in), static_cast<const T*>(k_in), static_cast<const T*>(v_in), ld,       \
      static_cast<T*>(k_cache), static_cast<T*>(v_cache), q_norm_weight, k_norm_weight, inv_freq, rot_mult,   \
      positions, slots, (int)H, (int)G, (int)dim, (int)vdim, (int)rot_dims, eps)
  switch (dtype) {
    case B200_BF16: DP_CALL(__nv_bfloat16); break;
    case B200_FP16: DP_CALL(__half); break;
    case B200_FP32: DP_CALL(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef DP_CALL
  B200_LAUNCH_OK("diff_attn_prepare_kernel");
  return B200_OK;
}

int b200_diff_attn(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                   const void* gate, int64_t ldg, const int32_t* q_cu_lens, const int32_t* kv_cu_lens,
                   const int32_t* block_tables, const int32_t* cu_block_lens, const int32_t* token_seq,
                   int64_t rows, int64_t H, int64_t G, int64_t dim, int64_t vdim, int64_t block_size, float scale,
                   int64_t window, int64_t keep_first, float lambda, float out_scale, float eps, int dtype,
                   b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens &&
                     token_seq, "diff_attn: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && H <= 65535 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 &&
                     vdim <= 32 * kMaxVPerLane && block_size > 0 && ldo >= H * vdim && window >= 0 &&
                     window < (1ll << 31) && keep_first >= 0 && keep_first < (1ll << 31),
                 "diff_attn: bad shape (value width at most 256; window 0 = every earlier key)");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(2 * dim + kWarps * 2 * vdim + kWarps * 4) * sizeof(float);
  B200_CHECK_ARG(smem <= 48 * 1024, "diff_attn: head too wide");
  dim3 grid((unsigned)rows, (unsigned)H);
#define DA_CALL(T)                                                                                             \
  diff_attn_kernel<T><<<grid, kWarps * 32, smem, st>>>(                                                        \
      static_cast<T*>(out), ldo, q, static_cast<const T*>(k_cache), static_cast<const T*>(v_cache),           \
      static_cast<const T*>(gate), ldg, q_cu_lens, kv_cu_lens, block_tables, cu_block_lens, token_seq, (int)H, \
      (int)G, (int)dim, (int)vdim, (int)block_size, scale, (int)window, (int)keep_first, lambda, out_scale, eps)
  switch (dtype) {
    case B200_BF16: DA_CALL(__nv_bfloat16); break;
    case B200_FP16: DA_CALL(__half); break;
    case B200_FP32: DA_CALL(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef DA_CALL
  B200_LAUNCH_OK("diff_attn_kernel");
  return B200_OK;
}

}  // extern "C"
