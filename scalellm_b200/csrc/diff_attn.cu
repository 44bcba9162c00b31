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
//   attend  : one CTA per (row, key/value head): its warps are the group's query heads times a split of the
//             visible keys; a warp walks its keys in groups of 32 (lane = key for the two scores, lane = value
//             channels for the weighted sum) with a running maximum and sum per map, and the splits of a head are
//             merged through shared memory.
// Scores, softmax weights, sums, the norm and the gate are fp32.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarps = 4;           // the per-token kernel
constexpr int kMaxWarps = 16;       // the attention kernel: heads of a group x key splits
constexpr int kMaxVdim = 512;

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

// One CTA per (row, key/value head, chunk of RH query heads of that group); warp = (head r, key split s), so the
// RH heads' reads of the same cache rows meet in L1.  NCH: value channels per lane = 4 * NCH (lane owns channels
// (c * 32 + lane) * 4 .. + 3 when VEC, lane + 32 * c otherwise).  VEC needs dim % 4 == 0 and vdim % 4 == 0 with
// 16-byte aligned map starts.
template <typename T, int NCH, bool VEC>
__global__ void __launch_bounds__(kMaxWarps * 32)
diff_attn_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ q, const T* __restrict__ k_cache,
                 const T* __restrict__ v_cache, const T* __restrict__ gate, int64_t ldg,
                 const int* __restrict__ q_cu, const int* __restrict__ kv_cu, const int* __restrict__ block_tables,
                 const int* __restrict__ cu_block_lens, const int* __restrict__ token_seq, int H, int G, int dim,
                 int vdim, int block_size, float scale, int window, int keep_first, float lambda, float out_scale,
                 float eps, int RH, int S) {
  extern __shared__ __align__(16) float sm[];
  const int n_warps = RH * S;
  float* q_s = sm;                                   // [RH][2 * dim]
  float* acc_s = q_s + RH * 2 * dim;                 // [n_warps][2][vdim]
  float* ml_s = acc_s + n_warps * 2 * vdim;          // [n_warps][4]  m1 l1 m2 l2
  const int row = blockIdx.x, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = H / G;
  const int r = warp % RH, sp = warp / RH;
  const int h_local = blockIdx.z * RH + r;           // head within the group
  const bool head_ok = h_local < R;
  const int h = g * R + (head_ok ? h_local : 0);
  const int seq = token_seq[row];
  const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
  const int i = kv_len - q_len + (row - q_cu[seq]);            // position of this row
  const int* table = block_tables + cu_block_lens[seq];
  for (int d = threadIdx.x; d < RH * 2 * dim; d += blockDim.x) {
    const int rr = d / (2 * dim), hh = blockIdx.z * RH + rr;
    q_s[d] = hh < R ? q[((size_t)row * H + g * R + hh) * 2 * dim + (d - rr * 2 * dim)] : 0.0f;
  }
  __syncthreads();
  const float* q1 = q_s + r * 2 * dim;
  const float* q2 = q1 + dim;
  // visible keys: the kept first tokens that have left the window, then the window
  const int lo = (window > 0 && i - window + 1 > 0) ? i - window + 1 : 0;
  const int ns = keep_first < lo ? keep_first : lo;
  const int total = ns + (i - lo + 1);
  const size_t k_stride = (size_t)G * 2 * dim, v_stride = (size_t)G * vdim;
  float m1 = -INFINITY, l1 = 0.0f, m2 = -INFINITY, l2 = 0.0f;
  float a1[4 * NCH], a2[4 * NCH];
#pragma unroll
  for (int c = 0; c < 4 * NCH; ++c) a1[c] = a2[c] = 0.0f;
  for (int n0 = sp * 32; n0 < total; n0 += S * 32) {
    const int n = n0 + lane;
    const bool live = n < total;
    float s1 = -INFINITY, s2 = -INFINITY;
    // lanes past the last key point at the row's own position (always written) with weight 0, so that the
    // weighted sum below runs over all 32 lanes without a test
    const int j = live ? (n < ns ? n : lo + (n - ns)) : i;
    const int slot = table[j / block_size] + j % block_size;
    if (live) {
      const T* kr = k_cache + (size_t)slot * k_stride + (size_t)g * 2 * dim;
      float d1 = 0.0f, d2 = 0.0f;
      if (VEC) {
        for (int d = 0; d < dim; d += 4) {
          float x[4], y[4];
          load4<T>(kr + d, x);
          load4<T>(kr + dim + d, y);
          const float4 u = *reinterpret_cast<const float4*>(q1 + d), w = *reinterpret_cast<const float4*>(q2 + d);
          d1 += u.x * x[0]; d1 += u.y * x[1]; d1 += u.z * x[2]; d1 += u.w * x[3];
          d2 += w.x * y[0]; d2 += w.y * y[1]; d2 += w.z * y[2]; d2 += w.w * y[3];
        }
      } else {
        for (int d = 0; d < dim; ++d) {
          d1 += q1[d] * Num<T>::to_f(kr[d]);
          d2 += q2[d] * Num<T>::to_f(kr[dim + d]);
        }
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
    for (int c = 0; c < 4 * NCH; ++c) { a1[c] *= c1; a2[c] *= c2; }
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      const float w1 = __shfl_sync(0xffffffffu, p1, kk), w2 = __shfl_sync(0xffffffffu, p2, kk);
      const int sl = __shfl_sync(0xffffffffu, slot, kk);
      const T* vr = v_cache + (size_t)sl * v_stride + (size_t)g * vdim;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        if (VEC) {
          const int col = (c * 32 + lane) * 4;
          if (col < vdim) {
            float v[4];
            load4<T>(vr + col, v);
#pragma unroll
            for (int e = 0; e < 4; ++e) { a1[c * 4 + e] += w1 * v[e]; a2[c * 4 + e] += w2 * v[e]; }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = lane + 32 * (c * 4 + e);
            if (col < vdim) {
              const float v = Num<T>::to_f(vr[col]);
              a1[c * 4 + e] += w1 * v;
              a2[c * 4 + e] += w2 * v;
            }
          }
        }
      }
    }
  }
  // merge the key splits of every head
  if (lane == 0) {
    ml_s[warp * 4 + 0] = m1; ml_s[warp * 4 + 1] = l1; ml_s[warp * 4 + 2] = m2; ml_s[warp * 4 + 3] = l2;
  }
  auto col_of = [&](int c, int e) { return VEC ? (c * 32 + lane) * 4 + e : lane + 32 * (c * 4 + e); };
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = col_of(c, e);
      if (col < vdim) {
        acc_s[(warp * 2 + 0) * vdim + col] = a1[c * 4 + e];
        acc_s[(warp * 2 + 1) * vdim + col] = a2[c * 4 + e];
      }
    }
  __syncthreads();
  if (sp != 0 || !head_ok) return;
  float M1 = -INFINITY, M2 = -INFINITY;
  for (int s2i = 0; s2i < S; ++s2i) {
    const int w = r + s2i * RH;
    M1 = fmaxf(M1, ml_s[w * 4]);
    M2 = fmaxf(M2, ml_s[w * 4 + 2]);
  }
  float L1 = 0.0f, L2 = 0.0f;
  float o[4 * NCH];
#pragma unroll
  for (int c = 0; c < 4 * NCH; ++c) o[c] = 0.0f;
  float x2[4 * NCH];
#pragma unroll
  for (int c = 0; c < 4 * NCH; ++c) x2[c] = 0.0f;
  for (int s2i = 0; s2i < S; ++s2i) {
    const int w = r + s2i * RH;
    const float f1 = ml_s[w * 4 + 1] > 0.0f ? expf(ml_s[w * 4] - M1) : 0.0f;
    const float f2 = ml_s[w * 4 + 3] > 0.0f ? expf(ml_s[w * 4 + 2] - M2) : 0.0f;
    L1 += f1 * ml_s[w * 4 + 1];
    L2 += f2 * ml_s[w * 4 + 3];
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = col_of(c, e);
        if (col < vdim) {
          o[c * 4 + e] += f1 * acc_s[(w * 2 + 0) * vdim + col];
          x2[c * 4 + e] += f2 * acc_s[(w * 2 + 1) * vdim + col];
        }
      }
  }
  float ss = 0.0f;
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (col_of(c, e) < vdim) {
        o[c * 4 + e] = o[c * 4 + e] / L1 - lambda * (x2[c * 4 + e] / L2);
        ss += o[c * 4 + e] * o[c * 4 + e];
      }
    }
  ss = warp_sum(ss);
  const float gl = gate ? 1.0f / (1.0f + expf(-Num<T>::to_f(gate[(size_t)row * ldg + h]))) : 1.0f;
  const float f = out_scale * gl / sqrtf(ss / (float)vdim + eps);
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = col_of(c, e);
      if (col < vdim) out[(size_t)row * ldo + (size_t)h * vdim + col] = Num<T>::from_f(o[c * 4 + e] * f);
    }
}

// The same walk with the keys and values of a tile brought into shared memory first: TK = 32 S keys per tile, copied
// asynchronously (16 bytes a piece, whole rows side by side) into one of two buffers while the other is consumed, so
// that the cache is read once per CTA in full lines and lane = key reads its row from shared memory (rows padded by 16
// bytes: no bank conflicts).  Needs K and V head rows that are multiples of 16 bytes.
__device__ __forceinline__ void cp_async16_plain(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

template <typename T, int NCH>
__global__ void __launch_bounds__(256)
diff_attn_staged_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ q, const T* __restrict__ k_cache,
                        const T* __restrict__ v_cache, const T* __restrict__ gate, int64_t ldg,
                        const int* __restrict__ q_cu, const int* __restrict__ kv_cu,
                        const int* __restrict__ block_tables, const int* __restrict__ cu_block_lens,
                        const int* __restrict__ token_seq, int H, int G, int dim, int vdim, int block_size,
                        float scale, int window, int keep_first, float lambda, float out_scale, float eps, int RH,
                        int S) {
  extern __shared__ __align__(16) float sm[];
  constexpr int EPC = 16 / (int)sizeof(T);           // elements per 16-byte piece
  const int n_warps = RH * S, TK = 32 * S;
  const int KROW = 2 * dim + EPC, VROW = vdim + EPC; // elements per staged row
  float* q_s = sm;                                   // [RH][2 * dim]
  float* acc_s = q_s + RH * 2 * dim;                 // [n_warps][2][vdim]
  float* ml_s = acc_s + n_warps * 2 * vdim;          // [n_warps][4]
  T* Kst = reinterpret_cast<T*>(ml_s + ((n_warps * 4 + 3) / 4) * 4);   // [2][TK][KROW]
  T* Vst = Kst + (size_t)2 * TK * KROW;                                // [2][TK][VROW]
  const int row = blockIdx.x, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = H / G;
  const int r = warp % RH, sp = warp / RH;
  const int h_local = blockIdx.z * RH + r;
  const bool head_ok = h_local < R;
  const int h = g * R + (head_ok ? h_local : 0);
  const int seq = token_seq[row];
  const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
  const int i = kv_len - q_len + (row - q_cu[seq]);
  const int* table = block_tables + cu_block_lens[seq];
  for (int d = threadIdx.x; d < RH * 2 * dim; d += blockDim.x) {
    const int rr = d / (2 * dim), hh = blockIdx.z * RH + rr;
    q_s[d] = hh < R ? q[((size_t)row * H + g * R + hh) * 2 * dim + (d - rr * 2 * dim)] : 0.0f;
  }
  const int lo = (window > 0 && i - window + 1 > 0) ? i - window + 1 : 0;
  const int ns = keep_first < lo ? keep_first : lo;
  const int total = ns + (i - lo + 1);
  const int n_tiles = (total + TK - 1) / TK;
  const size_t k_stride = (size_t)G * 2 * dim, v_stride = (size_t)G * vdim;
  const int kp = 2 * dim / EPC, vp = vdim / EPC;     // 16-byte pieces per key row and value row
  auto load_tile = [&](int idx, int buf) {
    for (int key = warp; key < TK; key += n_warps) {
      const int n = idx * TK + key;
      // keys past the last one stand in as the row's own position (always written) and get weight 0
      const int j = n < total ? (n < ns ? n : lo + (n - ns)) : i;
      const size_t slot = (size_t)table[j / block_size] + j % block_size;
      const T* kr = k_cache + slot * k_stride + (size_t)g * 2 * dim;
      const T* vr = v_cache + slot * v_stride + (size_t)g * vdim;
      T* kd = Kst + ((size_t)buf * TK + key) * KROW;
      T* vd = Vst + ((size_t)buf * TK + key) * VROW;
      for (int c = lane; c < kp + vp; c += 32) {
        if (c < kp) cp_async16_plain(kd + c * EPC, kr + c * EPC);
        else cp_async16_plain(vd + (c - kp) * EPC, vr + (c - kp) * EPC);
      }
    }
  };
  load_tile(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  const float* q1 = q_s + r * 2 * dim;
  const float* q2 = q1 + dim;
  float m1 = -INFINITY, l1 = 0.0f, m2 = -INFINITY, l2 = 0.0f;
  float a1[4 * NCH], a2[4 * NCH];
#pragma unroll
  for (int c = 0; c < 4 * NCH; ++c) a1[c] = a2[c] = 0.0f;
  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (it + 1 < n_tiles) load_tile(it + 1, buf ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int n0 = it * TK + sp * 32;
    if (n0 >= total) continue;                         // this split has no key in the last tile
    const bool live = n0 + lane < total;
    const T* kr = Kst + ((size_t)buf * TK + sp * 32 + lane) * KROW;
    float s1 = -INFINITY, s2 = -INFINITY;
    if (live) {
      float d1 = 0.0f, d2 = 0.0f;
      for (int d = 0; d < dim; d += 4) {
        float x[4], y[4];
        load4<T>(kr + d, x);
        load4<T>(kr + dim + d, y);
        const float4 u = *reinterpret_cast<const float4*>(q1 + d), w = *reinterpret_cast<const float4*>(q2 + d);
        d1 += u.x * x[0]; d1 += u.y * x[1]; d1 += u.z * x[2]; d1 += u.w * x[3];
        d2 += w.x * y[0]; d2 += w.y * y[1]; d2 += w.z * y[2]; d2 += w.w * y[3];
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
    const float nm1 = fmaxf(m1, t1), nm2 = fmaxf(m2, t2);
    const float c1 = expf(m1 - nm1), c2 = expf(m2 - nm2);
    const float p1 = live ? expf(s1 - nm1) : 0.0f, p2 = live ? expf(s2 - nm2) : 0.0f;
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
    m1 = nm1;
    m2 = nm2;
#pragma unroll
    for (int c = 0; c < 4 * NCH; ++c) { a1[c] *= c1; a2[c] *= c2; }
    const T* vbase = Vst + ((size_t)buf * TK + sp * 32) * VROW;
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
      const float w1 = __shfl_sync(0xffffffffu, p1, kk), w2 = __shfl_sync(0xffffffffu, p2, kk);
      const T* vr = vbase + (size_t)kk * VROW;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = (c * 32 + lane) * 4;
        if (col < vdim) {
          float v[4];
          load4<T>(vr + col, v);
#pragma unroll
          for (int e = 0; e < 4; ++e) { a1[c * 4 + e] += w1 * v[e]; a2[c * 4 + e] += w2 * v[e]; }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (lane == 0) {
    ml_s[warp * 4 + 0] = m1; ml_s[warp * 4 + 1] = l1; ml_s[warp * 4 + 2] = m2; ml_s[warp * 4 + 3] = l2;
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = (c * 32 + lane) * 4 + e;
      if (col < vdim) {
        acc_s[(warp * 2 + 0) * vdim + col] = a1[c * 4 + e];
        acc_s[(warp * 2 + 1) * vdim + col] = a2[c * 4 + e];
      }
    }
  __syncthreads();
  if (sp != 0 || !head_ok) return;
  float M1 = -INFINITY, M2 = -INFINITY;
  for (int k = 0; k < S; ++k) {
    M1 = fmaxf(M1, ml_s[(r + k * RH) * 4]);
    M2 = fmaxf(M2, ml_s[(r + k * RH) * 4 + 2]);
  }
  float L1 = 0.0f, L2 = 0.0f, o[4 * NCH], x2[4 * NCH];
#pragma unroll
  for (int c = 0; c < 4 * NCH; ++c) o[c] = x2[c] = 0.0f;
  for (int k = 0; k < S; ++k) {
    const int w = r + k * RH;
    const float f1 = ml_s[w * 4 + 1] > 0.0f ? expf(ml_s[w * 4] - M1) : 0.0f;
    const float f2 = ml_s[w * 4 + 3] > 0.0f ? expf(ml_s[w * 4 + 2] - M2) : 0.0f;
    L1 += f1 * ml_s[w * 4 + 1];
    L2 += f2 * ml_s[w * 4 + 3];
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = (c * 32 + lane) * 4 + e;
        if (col < vdim) {
          o[c * 4 + e] += f1 * acc_s[(w * 2 + 0) * vdim + col];
          x2[c * 4 + e] += f2 * acc_s[(w * 2 + 1) * vdim + col];
        }
      }
  }
  float ss = 0.0f;
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if ((c * 32 + lane) * 4 + e < vdim) {
        o[c * 4 + e] = o[c * 4 + e] / L1 - lambda * (x2[c * 4 + e] / L2);
        ss += o[c * 4 + e] * o[c * 4 + e];
      }
  ss = warp_sum(ss);
  const float gl = gate ? 1.0f / (1.0f + expf(-Num<T>::to_f(gate[(size_t)row * ldg + h]))) : 1.0f;
  const float f = out_scale * gl / sqrtf(ss / (float)vdim + eps);
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = (c * 32 + lane) * 4 + e;
      if (col < vdim) out[(size_t)row * ldo + (size_t)h * vdim + col] = Num<T>::from_f(o[c * 4 + e] * f);
    }
}

// ------------------------------------------------------------------------------------------------------------
// Prompt portions in bf16 on the tensor cores (mma.sync m16n8k16, fp32 accumulation).
// One CTA = 4 warps = RW query heads of one key/value group x (4 / RW) sub-tiles of 16 consecutive tokens of one
// sequence, so that all warps walk the same key tiles: 32 keys per tile, K [32][2 dim] and V [32][vdim] copied
// asynchronously (two buffers) through the block table.  Per warp and tile: S1 = Q1 K1^T, S2 = Q2 K2^T, the
// visibility test per element, a running maximum / sum per row and map in fp32, and O1 += P1 V, O2 += P2 V with
// the weights entering the product as two bf16 terms (p = hi + lo, 16 mantissa bits).  The tiles visited are those
// that hold kept first tokens and those of the window of the CTA's tokens.
// ------------------------------------------------------------------------------------------------------------
constexpr int kBK = 32;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = smem_u32(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
  hi = Num<__nv_bfloat16>::pack(__bfloat162float(xh), __bfloat162float(yh));
  lo = Num<__nv_bfloat16>::pack(x - __bfloat162float(xh), y - __bfloat162float(yh));
}

// dim <= 16 KS_MAX, vdim <= 16 VT_MAX, both multiples of 16; EXACT: dim = 16 KS_MAX and vdim = 16 VT_MAX, known to
// the compiler (row pitches and fragment offsets become immediates, the loops lose their tests)
template <int KS_MAX, int VT_MAX, bool EXACT>
__global__ void __launch_bounds__(128)
diff_attn_prefill_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const float* __restrict__ q,
                         const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                         const __nv_bfloat16* __restrict__ gate, int64_t ldg, const int* __restrict__ q_cu,
                         const int* __restrict__ kv_cu, const int* __restrict__ block_tables,
                         const int* __restrict__ cu_block_lens, int H, int G, int dim_rt, int vdim_rt, int block_size,
                         float scale, int window, int keep_first, float lambda, float out_scale, float eps, int RW,
                         int chunks) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int dim = EXACT ? 16 * KS_MAX : dim_rt, vdim = EXACT ? 16 * VT_MAX : vdim_rt;
  const int KROW = 2 * dim + 8, VROW = vdim + 8;        // bf16 elements per staged row (16 bytes of padding)
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);     // [4][16][KROW]
  __nv_bfloat16* Ks = Qs + 4 * 16 * KROW;                          // [2][kBK][KROW]
  __nv_bfloat16* Vs = Ks + 2 * kBK * KROW;                         // [2][kBK][VROW]
  const int seq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.z / chunks, chunk = blockIdx.z % chunks;
  const int R = H / G, TW = 4 / RW, BQ = 16 * TW;
  const int q0 = q_cu[seq], q_len = q_cu[seq + 1] - q0, kv_len = kv_cu[seq + 1] - kv_cu[seq];
  const int t0 = blockIdx.x * BQ;                      // first token of the CTA within the step's portion
  if (t0 >= q_len) return;
  const int first_pos = kv_len - q_len;
  const int hr = warp % RW, ts = warp / RW;
  const int h_local = chunk * RW + hr;
  const bool head_ok = h_local < R;
  const int h = g * R + (head_ok ? h_local : 0);
  const int KS = dim / 16, VT = vdim / 16;
  const int* table = block_tables + cu_block_lens[seq];
  // stage this warp's 16 query rows (both maps) as bf16
  {
    __nv_bfloat16* qw = Qs + warp * 16 * KROW;
    for (int e = lane; e < 16 * 2 * dim; e += 32) {
      const int rr = e / (2 * dim), d = e - rr * 2 * dim;
      const int t = t0 + ts * 16 + rr;
      const float v = (t < q_len && head_ok) ? q[((size_t)(q0 + t) * H + h) * 2 * dim + d] : 0.0f;
      qw[rr * KROW + d] = __float2bfloat16_rn(v);
    }
  }
  // key tiles of the CTA: positions P0 .. P1 of its tokens
  const int P0 = first_pos + t0;
  const int P1 = first_pos + (t0 + BQ < q_len ? t0 + BQ : q_len) - 1;
  const int lo = (window > 0 && P0 - window + 1 > 0) ? P0 - window + 1 : 0;
  const int ns = keep_first < lo ? keep_first : lo;
  const int sink_tiles = (ns + kBK - 1) / kBK;
  const int wt0 = lo / kBK > sink_tiles ? lo / kBK : sink_tiles;
  const int n_tiles = sink_tiles + (P1 / kBK - wt0 + 1);
  auto tile_j0 = [&](int idx) { return (idx < sink_tiles ? idx : wt0 + idx - sink_tiles) * kBK; };
  const size_t k_stride = (size_t)G * 2 * dim, v_stride = (size_t)G * vdim;
  auto load_tile = [&](int idx, int buf) {
    const int j0 = tile_j0(idx);
    const int key = threadIdx.x >> 2, sub = threadIdx.x & 3;
    const int j = j0 + key;
    const bool ok = j <= P1;
    size_t slot = 0;
    if (ok) slot = (size_t)table[j / block_size] + j % block_size;
    const __nv_bfloat16* kr = k_cache + slot * k_stride + (size_t)g * 2 * dim;
    const __nv_bfloat16* vr = v_cache + slot * v_stride + (size_t)g * vdim;
    __nv_bfloat16* kd = Ks + ((size_t)buf * kBK + key) * KROW;
    __nv_bfloat16* vd = Vs + ((size_t)buf * kBK + key) * VROW;
    for (int c = sub; c < dim / 4; c += 4) cp_async16(kd + c * 8, kr + c * 8, ok);
    for (int c = sub; c < vdim / 8; c += 4) cp_async16(vd + c * 8, vr + c * 8, ok);
  };
  load_tile(0, 0);
  cp_async_commit();

  const int gr = lane >> 2, qc = (lane & 3) * 2;      // fragment row within 8, first column of the pair
  const int row_t[2] = {t0 + ts * 16 + gr, t0 + ts * 16 + gr + 8};
  int pos[2];
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) pos[r2] = (row_t[r2] < q_len && head_ok) ? first_pos + row_t[r2] : -1;
  const int wpos0 = first_pos + t0 + ts * 16;          // position of the warp's first row
  const bool warp_rows_valid = head_ok && t0 + ts * 16 + 15 < q_len;
  float mx[2][2], ls[2][2];                            // [map][row]
  float o[2][VT_MAX * 2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    mx[m][0] = mx[m][1] = -INFINITY;
    ls[m][0] = ls[m][1] = 0.0f;
#pragma unroll
    for (int n = 0; n < VT_MAX * 2; ++n) o[m][n][0] = o[m][n][1] = o[m][n][2] = o[m][n][3] = 0.0f;
  }
  const __nv_bfloat16* qw = Qs + warp * 16 * KROW;
  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it & 1;
    cp_async_wait_all();
    __syncthreads();                                   // tile `it` has landed; everyone is done with tile it - 1
    if (it + 1 < n_tiles) load_tile(it + 1, buf ^ 1);
    cp_async_commit();
    const int j0 = tile_j0(it);
    // every key of the tile visible from every row of this warp: all 16 rows valid, the tile's last key not after
    // the warp's first row, and its first key inside the window of the warp's last row (or the tile all kept)
    const bool full_tile = warp_rows_valid && j0 + kBK - 1 <= wpos0 &&
                           (window <= 0 || wpos0 + 15 - j0 < window || j0 + kBK - 1 < keep_first);
    const __nv_bfloat16* kt = Ks + (size_t)buf * kBK * KROW;
    const __nv_bfloat16* vt = Vs + (size_t)buf * kBK * VROW;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      float sc[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < KS_MAX; ++ks) {
        if (ks < KS) {
          uint32_t a[4];
          ldsm_x4(a, qw + (lane & 15) * KROW + m * dim + ks * 16 + (lane >> 4) * 8);
#pragma unroll
          for (int np = 0; np < 2; ++np) {             // two n-tiles (16 keys) per load
            uint32_t b[4];
            ldsm_x4(b, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * KROW + m * dim + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(sc[np * 2], a, b[0], b[1]);
            mma_bf16(sc[np * 2 + 1], a, b[2], b[3]);
          }
        }
      }
      // visibility (tested per element only on tiles that some row of the warp sees in part), running maximum
      float rmax[2] = {-INFINITY, -INFINITY};
      if (full_tile) {
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            sc[n][e] *= scale;
            rmax[e >> 1] = fmaxf(rmax[e >> 1], sc[n][e]);
          }
      } else {
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = j0 + n * 8 + qc + (e & 1), i = pos[e >> 1];
            const bool vis = j <= i && (window <= 0 || i - j < window || j < keep_first);
            const float v = vis ? sc[n][e] * scale : -INFINITY;
            sc[n][e] = v;
            rmax[e >> 1] = fmaxf(rmax[e >> 1], v);
          }
      }
      float corr[2], msafe[2];
#pragma unroll
      for (int r2 = 0; r2 < 2; ++r2) {
        rmax[r2] = fmaxf(rmax[r2], __shfl_xor_sync(0xffffffffu, rmax[r2], 1));
        rmax[r2] = fmaxf(rmax[r2], __shfl_xor_sync(0xffffffffu, rmax[r2], 2));
        const float nm = fmaxf(mx[m][r2], rmax[r2]);
        msafe[r2] = nm == -INFINITY ? 0.0f : nm;
        corr[r2] = __expf(mx[m][r2] - msafe[r2]);
        mx[m][r2] = nm;
        ls[m][r2] *= corr[r2];
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {   // the maximum settles after a few tiles
#pragma unroll
        for (int n = 0; n < VT_MAX * 2; ++n) {
          o[m][n][0] *= corr[0]; o[m][n][1] *= corr[0];
          o[m][n][2] *= corr[1]; o[m][n][3] *= corr[1];
        }
      }
      uint32_t phi[2][4], plo[2][4];                   // A fragments of the two 16-key steps
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const float p0 = __expf(sc[n][0] - msafe[0]), p1 = __expf(sc[n][1] - msafe[0]);   // 2 ulp: the products are bf16
        const float p2 = __expf(sc[n][2] - msafe[1]), p3 = __expf(sc[n][3] - msafe[1]);
        ls[m][0] += p0 + p1;
        ls[m][1] += p2 + p3;
        const int kk = n >> 1, half = (n & 1) * 2;
        split_bf16(p0, p1, phi[kk][half], plo[kk][half]);
        split_bf16(p2, p3, phi[kk][half + 1], plo[kk][half + 1]);
      }
      // four independent accumulators between two products into the same one (hi terms of a 32-channel strip,
      // then its lo terms)
#pragma unroll
      for (int kk = 0; kk < 2; ++kk)
#pragma unroll
        for (int vp = 0; vp < VT_MAX; vp += 2) {
          if (vp < VT) {
            const bool two = vp + 1 < VT;
            uint32_t b0[4], b1[4] = {0u, 0u, 0u, 0u};
            const __nv_bfloat16* vrow = vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VROW + (lane >> 4) * 8;
            ldsm_x4_t(b0, vrow + vp * 16);
            if (two) ldsm_x4_t(b1, vrow + (vp + 1) * 16);
            mma_bf16(o[m][vp * 2], phi[kk], b0[0], b0[1]);
            mma_bf16(o[m][vp * 2 + 1], phi[kk], b0[2], b0[3]);
            if (two) {
              mma_bf16(o[m][vp * 2 + 2], phi[kk], b1[0], b1[1]);
              mma_bf16(o[m][vp * 2 + 3], phi[kk], b1[2], b1[3]);
            }
            mma_bf16(o[m][vp * 2], plo[kk], b0[0], b0[1]);
            mma_bf16(o[m][vp * 2 + 1], plo[kk], b0[2], b0[3]);
            if (two) {
              mma_bf16(o[m][vp * 2 + 2], plo[kk], b1[0], b1[1]);
              mma_bf16(o[m][vp * 2 + 3], plo[kk], b1[2], b1[3]);
            }
          }
        }
    }
  }
  cp_async_wait_all();
  // rows: sums over the quad, the difference of the maps, the head's root mean square, the gate
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      ls[m][r2] += __shfl_xor_sync(0xffffffffu, ls[m][r2], 1);
      ls[m][r2] += __shfl_xor_sync(0xffffffffu, ls[m][r2], 2);
    }
  float ss[2] = {0.0f, 0.0f};
#pragma unroll
  for (int n = 0; n < VT_MAX * 2; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r2 = e >> 1;
      const float d = (n < VT * 2) ? o[0][n][e] / ls[0][r2] - lambda * (o[1][n][e] / ls[1][r2]) : 0.0f;
      o[0][n][e] = d;
      ss[r2] += d * d;
    }
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    ss[r2] += __shfl_xor_sync(0xffffffffu, ss[r2], 1);
    ss[r2] += __shfl_xor_sync(0xffffffffu, ss[r2], 2);
    if (pos[r2] < 0) continue;
    const size_t row = (size_t)q0 + row_t[r2];
    const float gl = gate ? 1.0f / (1.0f + expf(-__bfloat162float(gate[row * ldg + h]))) : 1.0f;
    const float f = out_scale * gl / sqrtf(ss[r2] / (float)vdim + eps);
    __nv_bfloat16* dst = out + row * ldo + (size_t)h * vdim;
#pragma unroll
    for (int n = 0; n < VT_MAX * 2; ++n)
      if (n < VT * 2)
        *reinterpret_cast<uint32_t*>(dst + n * 8 + qc) =
            Num<__nv_bfloat16>::pack(o[0][n][r2 * 2] * f, o[0][n][r2 * 2 + 1] * f);
  }
}

// ------------------------------------------------------------------------------------------------------------
// Single tokens in bf16 on the tensor cores: the 16 rows of the product are the query HEADS of one key/value group
// (all at the row's position), so one pass over the group's keys serves every head that shares them.  One CTA per
// (row, group[, chunk of 16 heads]); tiles of 64 keys are staged as above and each of the 4 warps takes 16 keys of
// every tile with accumulators of its own; the warps' running maxima, sums and weighted sums are merged through
// shared memory at the end.  A row's tiles may be shared out over n_splits such CTAs (few rows, many SMs): each then
// hands its merged sums to diff_attn_merge_kernel through a workspace.
// ------------------------------------------------------------------------------------------------------------
constexpr int kDK = 64;
constexpr int kDS = 2;     // staged tiles: one in flight while one is consumed (a third bought nothing: the walk of a
                           // CTA is bound by its own instruction latency, and shared memory bounds the CTAs per SM)

template <int KS_MAX, int VT_MAX>
__global__ void __launch_bounds__(128)
diff_attn_decode_tc_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const float* __restrict__ q,
                           const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                           const __nv_bfloat16* __restrict__ gate, int64_t ldg, const int* __restrict__ q_cu,
                           const int* __restrict__ kv_cu, const int* __restrict__ block_tables,
                           const int* __restrict__ cu_block_lens, const int* __restrict__ token_seq, int H, int G,
                           int dim, int vdim, int block_size, float scale, int window, int keep_first, float lambda,
                           float out_scale, float eps, int n_splits, float* __restrict__ ws) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int KROW = 2 * dim + 8, VROW = vdim + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);     // [16][KROW]
  float* ml_s = reinterpret_cast<float*>(Qs + 16 * KROW);          // [4 warps][2 maps][2: m, l][16 rows]
  unsigned char* big = reinterpret_cast<unsigned char*>(ml_s + 4 * 2 * 2 * 16);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(big);       // [kDS][kDK][KROW]
  __nv_bfloat16* Vs = Ks + kDS * kDK * KROW;                         // [kDS][kDK][VROW]
  float* o_s = reinterpret_cast<float*>(big);                      // after the walk: [4 warps][2 maps][16][vdim]
  const int row = blockIdx.x / n_splits, split = blockIdx.x % n_splits, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = H / G, h_base = blockIdx.z * 16;
  const int n_heads = R - h_base < 16 ? R - h_base : 16;           // valid rows of the tile
  const int seq = token_seq[row];
  const int kv_len = kv_cu[seq + 1] - kv_cu[seq], q_len = q_cu[seq + 1] - q_cu[seq];
  const int i = kv_len - q_len + (row - q_cu[seq]);
  const int KS = dim / 16, VT = vdim / 16;
  const int* table = block_tables + cu_block_lens[seq];
  for (int e = threadIdx.x; e < 16 * 2 * dim; e += 128) {
    const int rr = e / (2 * dim), d = e - rr * 2 * dim;
    const float v = rr < n_heads ? q[((size_t)row * H + g * R + h_base + rr) * 2 * dim + d] : 0.0f;
    Qs[rr * KROW + d] = __float2bfloat16_rn(v);
  }
  const int lo = (window > 0 && i - window + 1 > 0) ? i - window + 1 : 0;
  const int ns = keep_first < lo ? keep_first : lo;
  const int sink_tiles = (ns + kDK - 1) / kDK;
  const int wt0 = lo / kDK > sink_tiles ? lo / kDK : sink_tiles;
  const int all_tiles = sink_tiles + (i / kDK - wt0 + 1);
  // this CTA's share of the row's tiles (n_splits CTAs per row; an empty share hands on sums of zero)
  const int per = (all_tiles + n_splits - 1) / n_splits;
  const int tile0 = split * per;
  const int n_tiles = all_tiles - tile0 < per ? (all_tiles - tile0 > 0 ? all_tiles - tile0 : 0) : per;
  auto tile_j0 = [&](int idx) {
    const int t = tile0 + idx;
    return (t < sink_tiles ? t : wt0 + t - sink_tiles) * kDK;
  };
  const size_t k_stride = (size_t)G * 2 * dim, v_stride = (size_t)G * vdim;
  auto load_tile = [&](int idx, int buf) {
    const int j0 = tile_j0(idx);
    const int sub = threadIdx.x & 1;
    for (int key = threadIdx.x >> 1; key < kDK; key += 64) {
      const int j = j0 + key;
      const bool ok = j <= i;
      size_t slot = 0;
      if (ok) slot = (size_t)table[j / block_size] + j % block_size;
      const __nv_bfloat16* kr = k_cache + slot * k_stride + (size_t)g * 2 * dim;
      const __nv_bfloat16* vr = v_cache + slot * v_stride + (size_t)g * vdim;
      __nv_bfloat16* kd = Ks + ((size_t)buf * kDK + key) * KROW;
      __nv_bfloat16* vd = Vs + ((size_t)buf * kDK + key) * VROW;
      for (int c = sub; c < dim / 4; c += 2) cp_async16(kd + c * 8, kr + c * 8, ok);
      for (int c = sub; c < vdim / 8; c += 2) cp_async16(vd + c * 8, vr + c * 8, ok);
    }
  };
  for (int t = 0; t < kDS - 1; ++t) {
    if (t < n_tiles) load_tile(t, t);
    cp_async_commit();
  }
  const int gr = lane >> 2, qc = (lane & 3) * 2;
  float mx[2][2], ls[2][2];
  float o[2][VT_MAX * 2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    mx[m][0] = mx[m][1] = -INFINITY;
    ls[m][0] = ls[m][1] = 0.0f;
#pragma unroll
    for (int n = 0; n < VT_MAX * 2; ++n) o[m][n][0] = o[m][n][1] = o[m][n][2] = o[m][n][3] = 0.0f;
  }
  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it % kDS;
    asm volatile("cp.async.wait_group %0;" ::"n"(kDS - 2) : "memory");   // tile `it` has landed
    __syncthreads();                                       // and everyone is done with tile it - 1
    if (it + kDS - 1 < n_tiles) load_tile(it + kDS - 1, (it + kDS - 1) % kDS);
    cp_async_commit();
    const int j0 = tile_j0(it) + warp * 16;              // this warp's 16 keys of the tile
    if (j0 > i) continue;                                // all after the row's position
    const __nv_bfloat16* kt = Ks + ((size_t)buf * kDK + warp * 16) * KROW;
    const __nv_bfloat16* vt = Vs + ((size_t)buf * kDK + warp * 16) * VROW;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      float sc[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < KS_MAX; ++ks) {
        if (ks < KS) {
          uint32_t a[4], b[4];
          ldsm_x4(a, Qs + (lane & 15) * KROW + m * dim + ks * 16 + (lane >> 4) * 8);
          ldsm_x4(b, kt + ((lane & 7) + (lane >> 4) * 8) * KROW + m * dim + ks * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(sc[0], a, b[0], b[1]);
          mma_bf16(sc[1], a, b[2], b[3]);
        }
      }
      float rmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + n * 8 + qc + (e & 1);
          const bool vis = j <= i && (window <= 0 || i - j < window || j < keep_first);
          const float v = vis ? sc[n][e] * scale : -INFINITY;
          sc[n][e] = v;
          rmax[e >> 1] = fmaxf(rmax[e >> 1], v);
        }
      float corr[2], msafe[2];
#pragma unroll
      for (int r2 = 0; r2 < 2; ++r2) {
        rmax[r2] = fmaxf(rmax[r2], __shfl_xor_sync(0xffffffffu, rmax[r2], 1));
        rmax[r2] = fmaxf(rmax[r2], __shfl_xor_sync(0xffffffffu, rmax[r2], 2));
        const float nm = fmaxf(mx[m][r2], rmax[r2]);
        msafe[r2] = nm == -INFINITY ? 0.0f : nm;
        corr[r2] = __expf(mx[m][r2] - msafe[r2]);
        mx[m][r2] = nm;
        ls[m][r2] *= corr[r2];
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int n = 0; n < VT_MAX * 2; ++n) {
          o[m][n][0] *= corr[0]; o[m][n][1] *= corr[0];
          o[m][n][2] *= corr[1]; o[m][n][3] *= corr[1];
        }
      }
      uint32_t phi[4], plo[4];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const float p0 = __expf(sc[n][0] - msafe[0]), p1 = __expf(sc[n][1] - msafe[0]);
        const float p2 = __expf(sc[n][2] - msafe[1]), p3 = __expf(sc[n][3] - msafe[1]);
        ls[m][0] += p0 + p1;
        ls[m][1] += p2 + p3;
        split_bf16(p0, p1, phi[n * 2], plo[n * 2]);
        split_bf16(p2, p3, phi[n * 2 + 1], plo[n * 2 + 1]);
      }
#pragma unroll
      for (int vt16 = 0; vt16 < VT_MAX; ++vt16) {
        if (vt16 < VT) {
          uint32_t b[4];
          ldsm_x4_t(b, vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * VROW + vt16 * 16 + (lane >> 4) * 8);
          mma_bf16(o[m][vt16 * 2], phi, b[0], b[1]);
          mma_bf16(o[m][vt16 * 2 + 1], phi, b[2], b[3]);
          mma_bf16(o[m][vt16 * 2], plo, b[0], b[1]);
          mma_bf16(o[m][vt16 * 2 + 1], plo, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait_all();
  __syncthreads();                                       // the tiles are done with: their memory takes the partial sums
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      ls[m][r2] += __shfl_xor_sync(0xffffffffu, ls[m][r2], 1);
      ls[m][r2] += __shfl_xor_sync(0xffffffffu, ls[m][r2], 2);
      if ((lane & 3) == 0) {
        ml_s[((warp * 2 + m) * 2 + 0) * 16 + gr + r2 * 8] = mx[m][r2];
        ml_s[((warp * 2 + m) * 2 + 1) * 16 + gr + r2 * 8] = ls[m][r2];
      }
    }
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < VT_MAX * 2; ++n)
      if (n < VT * 2) {
        float* dst = o_s + ((size_t)(warp * 2 + m) * 16) * vdim + n * 8 + qc;
        dst[(size_t)gr * vdim] = o[m][n][0];
        dst[(size_t)gr * vdim + 1] = o[m][n][1];
        dst[(size_t)(gr + 8) * vdim] = o[m][n][2];
        dst[(size_t)(gr + 8) * vdim + 1] = o[m][n][3];
      }
  __syncthreads();
  // warp w finishes heads w, w + 4, ...: lanes over the value channels
  for (int rr = warp; rr < n_heads; rr += 4) {
    float M[2] = {-INFINITY, -INFINITY}, L[2] = {0.0f, 0.0f}, f[2][4];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
      for (int w = 0; w < 4; ++w) M[m] = fmaxf(M[m], ml_s[((w * 2 + m) * 2 + 0) * 16 + rr]);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float lw = ml_s[((w * 2 + m) * 2 + 1) * 16 + rr];
        f[m][w] = lw > 0.0f ? expf(ml_s[((w * 2 + m) * 2 + 0) * 16 + rr] - M[m]) : 0.0f;
        L[m] += f[m][w] * lw;
      }
    }
    const int h = g * R + h_base + rr;
    if (ws) {
      // one of several CTAs of this row: hand on (M, L) per map and the two unnormalised sums; the merge kernel ends
      float* dst = ws + (((size_t)row * H + h) * n_splits + split) * (size_t)(4 + 2 * vdim);
      if (lane == 0) { dst[0] = M[0]; dst[1] = L[0]; dst[2] = M[1]; dst[3] = L[1]; }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col = lane + 32 * c;
        if (col < vdim) {
          float x1 = 0.0f, x2 = 0.0f;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            x1 += f[0][w] * o_s[((size_t)(w * 2 + 0) * 16 + rr) * vdim + col];
            x2 += f[1][w] * o_s[((size_t)(w * 2 + 1) * 16 + rr) * vdim + col];
          }
          dst[4 + col] = x1;
          dst[4 + vdim + col] = x2;
        }
      }
      continue;
    }
    float d[4], ss = 0.0f;                               // vdim <= 128: up to 4 channels per lane
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = lane + 32 * c;
      d[c] = 0.0f;
      if (col < vdim) {
        float x1 = 0.0f, x2 = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          x1 += f[0][w] * o_s[((size_t)(w * 2 + 0) * 16 + rr) * vdim + col];
          x2 += f[1][w] * o_s[((size_t)(w * 2 + 1) * 16 + rr) * vdim + col];
        }
        d[c] = x1 / L[0] - lambda * (x2 / L[1]);
        ss += d[c] * d[c];
      }
    }
    ss = warp_sum(ss);
    const float gl = gate ? 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)row * ldg + h]))) : 1.0f;
    const float fo = out_scale * gl / sqrtf(ss / (float)vdim + eps);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = lane + 32 * c;
      if (col < vdim) out[(size_t)row * ldo + (size_t)h * vdim + col] = __float2bfloat16_rn(d[c] * fo);
    }
  }
}

// The end of the walk for rows whose keys were shared out over n_splits CTAs: one warp per (row, head) merges the
// shares' maxima, sums and weighted sums, then the difference of the maps, the head's root mean square and the gate.
__global__ void __launch_bounds__(128)
diff_attn_merge_kernel(__nv_bfloat16* __restrict__ out, int64_t ldo, const float* __restrict__ ws,
                       const __nv_bfloat16* __restrict__ gate, int64_t ldg, int64_t n_pairs, int H, int vdim,
                       int n_splits, float lambda, float out_scale, float eps) {
  const int64_t pair = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);      // row * H + head
  const int lane = threadIdx.x & 31;
  if (pair >= n_pairs) return;
  const int64_t row = pair / H;
  const int h = (int)(pair - row * H);
  const float* src = ws + (size_t)pair * n_splits * (size_t)(4 + 2 * vdim);
  const size_t stride = (size_t)(4 + 2 * vdim);
  float M[2] = {-INFINITY, -INFINITY}, L[2] = {0.0f, 0.0f};
  for (int s = 0; s < n_splits; ++s) {
    M[0] = fmaxf(M[0], src[s * stride + 0]);
    M[1] = fmaxf(M[1], src[s * stride + 2]);
  }
  float x1[4] = {0.0f, 0.0f, 0.0f, 0.0f}, x2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int s = 0; s < n_splits; ++s) {
    const float* p = src + s * stride;
    const float f1 = p[1] > 0.0f ? expf(p[0] - M[0]) : 0.0f, f2 = p[3] > 0.0f ? expf(p[2] - M[1]) : 0.0f;
    L[0] += f1 * p[1];
    L[1] += f2 * p[3];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = lane + 32 * c;
      if (col < vdim) {
        x1[c] += f1 * p[4 + col];
        x2[c] += f2 * p[4 + vdim + col];
      }
    }
  }
  float d[4], ss = 0.0f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    d[c] = lane + 32 * c < vdim ? x1[c] / L[0] - lambda * (x2[c] / L[1]) : 0.0f;
    ss += d[c] * d[c];
  }
  ss = warp_sum(ss);
  const float gl = gate ? 1.0f / (1.0f + expf(-__bfloat162float(gate[row * ldg + h]))) : 1.0f;
  const float fo = out_scale * gl / sqrtf(ss / (float)vdim + eps);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int col = lane + 32 * c;
    if (col < vdim) out[row * ldo + (size_t)h * vdim + col] = __float2bfloat16_rn(d[c] * fo);
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
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && G <= 65535 && H % G == 0 && dim > 0 && vdim > 0 &&
                     vdim <= kMaxVdim && block_size > 0 && ldo >= H * vdim && window >= 0 &&
                     window < (1ll << 31) && keep_first >= 0 && keep_first < (1ll << 31),
                 "diff_attn: bad shape (value width at most 512; window 0 = every earlier key)");
  auto st = static_cast<cudaStream_t>(stream);
  const int R = (int)(H / G);
  const int RH = R < kMaxWarps ? R : kMaxWarps;     // query heads of the group per CTA
  const int S = kMaxWarps / RH;                     // key splits per head
  const int chunks = (R + RH - 1) / RH;
  const size_t smem = (size_t)(RH * 2 * dim + RH * S * 2 * vdim + RH * S * 4) * sizeof(float);
  B200_CHECK_ARG(smem <= 200 * 1024 && chunks <= 65535, "diff_attn: heads too wide");
  const int esz = dtype == B200_FP32 ? 4 : 2;
  const bool vec = dim % 4 == 0 && vdim % 4 == 0 && (dim * esz) % 16 == 0 && (vdim * esz) % 8 == 0 &&
                   is_aligned(k_cache, 16) && is_aligned(v_cache, 16);
  const int nch = vdim <= 128 ? 1 : (vdim <= 256 ? 2 : 4);
  dim3 grid((unsigned)rows, (unsigned)G, (unsigned)chunks);
  // rows of whole 16-byte pieces: the keys and values of a tile go through shared memory
  if (vec && (2 * dim * esz) % 16 == 0 && (vdim * esz) % 16 == 0) {
    const int RHs = R < 8 ? R : 8, Ss = 8 / RHs, TK = 32 * Ss, ch = (R + RHs - 1) / RHs, epc = 16 / esz;
    const size_t smem_s = (size_t)(RHs * 2 * dim + RHs * Ss * 2 * vdim + ((RHs * Ss * 4 + 3) / 4) * 4) * sizeof(float) +
                          (size_t)2 * TK * (2 * dim + epc + vdim + epc) * esz;
    if (smem_s <= 200 * 1024 && ch <= 65535) {
      dim3 grid_s((unsigned)rows, (unsigned)G, (unsigned)ch);
#define DAS_LAUNCH(T, NCH)                                                                                     \
  do {                                                                                                         \
    if (smem_s > 48 * 1024)                                                                                    \
      B200_CUDA_OK(cudaFuncSetAttribute(diff_attn_staged_kernel<T, NCH>,                                       \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s));            \
    diff_attn_staged_kernel<T, NCH><<<grid_s, RHs * Ss * 32, smem_s, st>>>(                                    \
        static_cast<T*>(out), ldo, q, static_cast<const T*>(k_cache), static_cast<const T*>(v_cache),         \
        static_cast<const T*>(gate), ldg, q_cu_lens, kv_cu_lens, block_tables, cu_block_lens, token_seq,      \
        (int)H, (int)G, (int)dim, (int)vdim, (int)block_size, scale, (int)window, (int)keep_first, lambda,    \
        out_scale, eps, RHs, Ss);                                                                              \
  } while (0)
#define DAS_CALL(T)                                                                                            \
  do {                                                                                                         \
    if (nch == 1) DAS_LAUNCH(T, 1); else if (nch == 2) DAS_LAUNCH(T, 2); else DAS_LAUNCH(T, 4);                \
  } while (0)
      switch (dtype) {
        case B200_BF16: DAS_CALL(__nv_bfloat16); break;
        case B200_FP16: DAS_CALL(__half); break;
        case B200_FP32: DAS_CALL(float); break;
        default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
      }
#undef DAS_CALL
#undef DAS_LAUNCH
      B200_LAUNCH_OK("diff_attn_staged_kernel");
      return B200_OK;
    }
  }
#define DA_LAUNCH(T, NCH, VEC)                                                                                 \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      B200_CUDA_OK(cudaFuncSetAttribute(diff_attn_kernel<T, NCH, VEC>,                                         \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));              \
    diff_attn_kernel<T, NCH, VEC><<<grid, RH * S * 32, smem, st>>>(                                            \
        static_cast<T*>(out), ldo, q, static_cast<const T*>(k_cache), static_cast<const T*>(v_cache),         \
        static_cast<const T*>(gate), ldg, q_cu_lens, kv_cu_lens, block_tables, cu_block_lens, token_seq,      \
        (int)H, (int)G, (int)dim, (int)vdim, (int)block_size, scale, (int)window, (int)keep_first, lambda,    \
        out_scale, eps, RH, S);                                                                                \
  } while (0)
#define DA_CALL(T)                                                                                             \
  do {                                                                                                         \
    if (vec) {                                                                                                 \
      if (nch == 1) DA_LAUNCH(T, 1, true); else if (nch == 2) DA_LAUNCH(T, 2, true); else DA_LAUNCH(T, 4, true); \
    } else {                                                                                                   \
      if (nch == 1) DA_LAUNCH(T, 1, false); else if (nch == 2) DA_LAUNCH(T, 2, false); else DA_LAUNCH(T, 4, false); \
    }                                                                                                          \
  } while (0)
  switch (dtype) {
    case B200_BF16: DA_CALL(__nv_bfloat16); break;
    case B200_FP16: DA_CALL(__half); break;
    case B200_FP32: DA_CALL(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef DA_CALL
#undef DA_LAUNCH
  B200_LAUNCH_OK("diff_attn_kernel");
  return B200_OK;
}

}  // extern "C"

extern "C" {

int b200_diff_attn_prefill_supported(int64_t dim, int64_t vdim, int dtype) {
  return dtype == B200_BF16 && dim > 0 && vdim > 0 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 128 && vdim <= 128;
}

int b200_diff_attn_prefill(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                           const void* gate, int64_t ldg, const int32_t* q_cu_lens, const int32_t* kv_cu_lens,
                           const int32_t* block_tables, const int32_t* cu_block_lens, int64_t n_seq, int64_t q_max,
                           int64_t H, int64_t G, int64_t dim, int64_t vdim, int64_t block_size, float scale,
                           int64_t window, int64_t keep_first, float lambda, float out_scale, float eps, int dtype,
                           b200_stream_t stream) {
  if (n_seq == 0 || q_max == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens,
                 "diff_attn_prefill: null pointer");
  if (!b200_diff_attn_prefill_supported(dim, vdim, dtype))
    return set_error(B200_ERR_UNSUPPORTED, "diff_attn_prefill: bf16 with dim and vdim multiples of 16 up to 128");
  B200_CHECK_ARG(n_seq > 0 && n_seq <= 65535 && q_max > 0 && H > 0 && G > 0 && H % G == 0 && block_size > 0 &&
                     ldo >= H * vdim && ldo % 2 == 0 && window >= 0 && window < (1ll << 31) && keep_first >= 0 &&
                     keep_first < (1ll << 31) && is_aligned(k_cache, 16) && is_aligned(v_cache, 16) &&
                     is_aligned(out, 4),
                 "diff_attn_prefill: bad shape or alignment");
  auto st = static_cast<cudaStream_t>(stream);
  const int R = (int)(H / G);
  const int RW = R >= 4 ? 4 : (R >= 2 ? 2 : 1);
  const int chunks = (R + RW - 1) / RW;
  const int BQ = 16 * (4 / RW);
  B200_CHECK_ARG(G * chunks <= 65535, "diff_attn_prefill: too many heads");
  const size_t smem = ((size_t)(4 * 16 + 2 * kBK) * (2 * dim + 8) + (size_t)2 * kBK * (vdim + 8)) * 2;
  dim3 grid((unsigned)((q_max + BQ - 1) / BQ), (unsigned)n_seq, (unsigned)(G * chunks));
#define DAP_LAUNCH(KS, VT, EX)                                                                                   \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      B200_CUDA_OK(cudaFuncSetAttribute(diff_attn_prefill_kernel<KS, VT, EX>,                                  \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));              \
    diff_attn_prefill_kernel<KS, VT, EX><<<grid, 128, smem, st>>>(                                                 \
        static_cast<__nv_bfloat16*>(out), ldo, q, static_cast<const __nv_bfloat16*>(k_cache),                  \
        static_cast<const __nv_bfloat16*>(v_cache), static_cast<const __nv_bfloat16*>(gate), ldg, q_cu_lens,   \
        kv_cu_lens, block_tables, cu_block_lens, (int)H, (int)G, (int)dim, (int)vdim, (int)block_size, scale,  \
        (int)window, (int)keep_first, lambda, out_scale, eps, RW, chunks);                                     \
  } while (0)
  if (dim == 64 && vdim == 128) DAP_LAUNCH(4, 8, true);          // common head shapes, sizes known to the compiler
  else if (dim == 128 && vdim == 128) DAP_LAUNCH(8, 8, true);
  else if (dim == 64 && vdim == 64) DAP_LAUNCH(4, 4, true);
  else if (dim == 32 && vdim == 64) DAP_LAUNCH(2, 4, true);
  else if (dim == 32 && vdim == 32) DAP_LAUNCH(2, 2, true);
  else if (dim <= 64 && vdim <= 64) DAP_LAUNCH(4, 4, false);
  else if (dim <= 64) DAP_LAUNCH(4, 8, false);
  else if (vdim <= 64) DAP_LAUNCH(8, 4, false);
  else DAP_LAUNCH(8, 8, false);
#undef DAP_LAUNCH
  B200_LAUNCH_OK("diff_attn_prefill_kernel");
  return B200_OK;
}

}  // extern "C"

extern "C" {

int b200_diff_attn_decode_tc(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                             const void* gate, int64_t ldg, const int32_t* q_cu_lens, const int32_t* kv_cu_lens,
                             const int32_t* block_tables, const int32_t* cu_block_lens, const int32_t* token_seq,
                             int64_t rows, int64_t H, int64_t G, int64_t dim, int64_t vdim, int64_t block_size,
                             float scale, int64_t window, int64_t keep_first, float lambda, float out_scale, float eps,
                             int64_t n_splits, float* workspace, int64_t workspace_floats, int dtype,
                             b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && q && k_cache && v_cache && q_cu_lens && kv_cu_lens && block_tables && cu_block_lens &&
                     token_seq, "diff_attn_decode_tc: null pointer");
  if (!b200_diff_attn_prefill_supported(dim, vdim, dtype))
    return set_error(B200_ERR_UNSUPPORTED, "diff_attn_decode_tc: bf16 with dim and vdim multiples of 16 up to 128");
  B200_CHECK_ARG(rows > 0 && H > 0 && G > 0 && G <= 65535 && H % G == 0 && block_size > 0 && ldo >= H * vdim &&
                     window >= 0 && window < (1ll << 31) && keep_first >= 0 && keep_first < (1ll << 31) &&
                     is_aligned(k_cache, 16) && is_aligned(v_cache, 16),
                 "diff_attn_decode_tc: bad shape or alignment");
  auto st = static_cast<cudaStream_t>(stream);
  const int R = (int)(H / G), chunks = (R + 15) / 16;
  const size_t tiles = ((size_t)kDS * kDK * (2 * dim + 8) + (size_t)kDS * kDK * (vdim + 8)) * 2;
  const size_t merge = (size_t)4 * 2 * 16 * vdim * sizeof(float);
  const size_t big = tiles > merge ? tiles : merge;
  const size_t smem = (size_t)16 * (2 * dim + 8) * 2 + 4 * 2 * 2 * 16 * sizeof(float) + big;
  B200_CHECK_ARG(n_splits >= 1 && n_splits <= 64 && rows * n_splits < (1ll << 31) &&
                     (n_splits == 1 || (workspace && workspace_floats >= rows * H * n_splits * (4 + 2 * vdim))),
                 "diff_attn_decode_tc: 1..64 key splits; more than one needs rows * H * splits * (4 + 2 vdim) floats");
  float* ws = n_splits > 1 ? workspace : nullptr;
  dim3 grid((unsigned)(rows * n_splits), (unsigned)G, (unsigned)chunks);
#define DAD_LAUNCH(KS, VT)                                                                                     \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      B200_CUDA_OK(cudaFuncSetAttribute(diff_attn_decode_tc_kernel<KS, VT>,                                    \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));              \
    diff_attn_decode_tc_kernel<KS, VT><<<grid, 128, smem, st>>>(                                               \
        static_cast<__nv_bfloat16*>(out), ldo, q, static_cast<const __nv_bfloat16*>(k_cache),                  \
        static_cast<const __nv_bfloat16*>(v_cache), static_cast<const __nv_bfloat16*>(gate), ldg, q_cu_lens,   \
        kv_cu_lens, block_tables, cu_block_lens, token_seq, (int)H, (int)G, (int)dim, (int)vdim,               \
        (int)block_size, scale, (int)window, (int)keep_first, lambda, out_scale, eps, (int)n_splits, ws);      \
  } while (0)
  if (dim <= 64 && vdim <= 64) DAD_LAUNCH(4, 4);
  else if (dim <= 64) DAD_LAUNCH(4, 8);
  else if (vdim <= 64) DAD_LAUNCH(8, 4);
  else DAD_LAUNCH(8, 8);
#undef DAD_LAUNCH
  B200_LAUNCH_OK("diff_attn_decode_tc_kernel");
  if (ws) {
    const int64_t n_pairs = rows * H;
    diff_attn_merge_kernel<<<(unsigned)((n_pairs + 3) / 4), 128, 0, st>>>(
        static_cast<__nv_bfloat16*>(out), ldo, ws, static_cast<const __nv_bfloat16*>(gate), ldg, n_pairs, (int)H,
        (int)vdim, (int)n_splits, lambda, out_scale, eps);
    B200_LAUNCH_OK("diff_attn_merge_kernel");
  }
  return B200_OK;
}

}  // extern "C"
