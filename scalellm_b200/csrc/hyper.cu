// hyper.cu — residual-stream kernels for decoders that keep several residual streams in fp32
// (hyper-connections), normalise with an offset RMS norm, mix each token with its predecessor
// (token shift) and gate every sublayer's result before it enters the streams.
//
//   X        [rows, S, W] fp32          the S residual streams of every token of the step
//   collapse u = sum_s a[s] X[., s, :]  (a == nullptr: plain sum)
//   norm     n = u * rsqrt(mean(u^2) + eps) * (offset + w)
//   shift    h_t = n_t + (n_{t-1} - n_t) * mu   with n_{-1} = 0 and n_{t-1} taken from the
//            sequence's state slot when token t opens a step's portion
//   update   X[., t, :] <- sum_s M[s, t] X[., s, :] + b[t] * y * sigmoid(g + c)
//
// All reductions, the streams and the state are fp32; T is the activation type (bf16 / fp16 / fp32).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kMaxStreams = 8;
constexpr int kRowThreads = 256;

template <typename T>
__global__ void embed_streams_kernel(float* __restrict__ X, const T* __restrict__ table,
                                     const int* __restrict__ tokens, int W, int S, int vocab) {
  const int row = blockIdx.x;
  int tok = tokens[row];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const T* src = table + (size_t)tok * W;
  float* dst = X + (size_t)row * S * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = Num<T>::to_f(src[i]);
    for (int s = 0; s < S; ++s) dst[(size_t)s * W + i] = v;
  }
}

// one CTA per row; the collapsed row is held in shared memory between the two passes
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
hc_norm_kernel(T* __restrict__ out, float* __restrict__ out32, const float* __restrict__ X,
               const float* __restrict__ a, const float* __restrict__ w, int W, int S, float eps,
               float offset) {
  extern __shared__ float u_s[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  const float* x = X + (size_t)row * S * W;
  float coef[kMaxStreams];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) coef[s] = (s < S) ? (a ? a[s] : 1.0f) : 0.0f;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    float u = 0.0f;
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < S) u += coef[s] * x[(size_t)s * W + i];
    u_s[i] = u;
    ss += u * u;
  }
  ss = block_sum<kRowThreads>(ss, red);
  const float r = rsqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    const float n = u_s[i] * r * (offset + w[i]);
    out[(size_t)row * W + i] = Num<T>::from_f(n);
    if (out32) out32[(size_t)row * W + i] = n;
  }
}

// one CTA per row.  The CTA of a portion's first row reads the sequence's state slot and is the
// only writer of that slot (it stores the portion's last unshifted row), so no other CTA races it.
template <typename T>
__global__ void token_shift_kernel(T* __restrict__ out, const float* __restrict__ n32,
                                   const float* __restrict__ mu, float* __restrict__ state,
                                   const int* __restrict__ q_cu, const int* __restrict__ positions,
                                   const int* __restrict__ token_seq,
                                   const int* __restrict__ state_slots, int W) {
  const int row = blockIdx.x;
  const int seq = token_seq[row];
  const int first = q_cu[seq], last = q_cu[seq + 1] - 1;
  const float* cur = n32 + (size_t)row * W;
  if (row != first) {
    const float* prev = cur - W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float n = cur[i];
      out[(size_t)row * W + i] = Num<T>::from_f(n + (prev[i] - n) * mu[i]);
    }
    return;
  }
  float* slot = state + (size_t)state_slots[seq] * W;
  const bool fresh = positions[row] == 0;
  const float* tail = n32 + (size_t)last * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float n = cur[i];
    const float p = fresh ? 0.0f : slot[i];
    out[(size_t)row * W + i] = Num<T>::from_f(n + (p - n) * mu[i]);
    slot[i] = tail[i];
  }
}

template <typename T>
__global__ void gated_hc_update_kernel(float* __restrict__ X, const T* __restrict__ y,
                                       const T* __restrict__ gate, const float* __restrict__ gate_bias,
                                       const float* __restrict__ mix, const float* __restrict__ outc,
                                       int W, int S, int64_t ldy, int64_t ldg) {
  const int row = blockIdx.x;
  float* x = X + (size_t)row * S * W;
  __shared__ float m_s[kMaxStreams * kMaxStreams + kMaxStreams];
  if (threadIdx.x < S * S) m_s[threadIdx.x] = mix ? mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.0f : 0.0f);
  if (threadIdx.x < S) m_s[kMaxStreams * kMaxStreams + threadIdx.x] = outc ? outc[threadIdx.x] : 1.0f;
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = Num<T>::to_f(y[(size_t)row * ldy + i]);
    if (gate) {
      const float z = Num<T>::to_f(gate[(size_t)row * ldg + i]) + (gate_bias ? gate_bias[i] : 0.0f);
      v *= 1.0f / (1.0f + expf(-z));
    }
    float old[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s)
      if (s < S) old[s] = x[(size_t)s * W + i];
#pragma unroll
    for (int t = 0; t < kMaxStreams; ++t) {
      if (t < S) {
        float acc = 0.0f;
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s)
          if (s < S) acc += m_s[s * S + t] * old[s];
        x[(size_t)t * W + i] = acc + m_s[kMaxStreams * kMaxStreams + t] * v;
      }
    }
  }
}


// ---- four columns per thread (W % 4 == 0): the same arithmetic with 16-byte accesses to the fp32 streams
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = Num<T>::to_f(p[i]);
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = Num<__nv_bfloat16>::unpack(u.x), b = Num<__nv_bfloat16>::unpack(u.y);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 u = *reinterpret_cast<const float4*>(p);
  v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = Num<T>::from_f(v[i]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 u;
  u.x = Num<__nv_bfloat16>::pack(v[0], v[1]);
  u.y = Num<__nv_bfloat16>::pack(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = u;
}
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
hc_norm_vec_kernel(T* __restrict__ out, float* __restrict__ out32, const float* __restrict__ X,
                   const float* __restrict__ a, const float* __restrict__ w, int W, int S, float eps,
                   float offset) {
  extern __shared__ __align__(16) float u_s[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  const float* x = X + (size_t)row * S * W;
  float coef[kMaxStreams];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) coef[s] = (s < S) ? (a ? a[s] : 1.0f) : 0.0f;
  float ss = 0.0f;
  for (int i = threadIdx.x * 4; i < W; i += kRowThreads * 4) {
    float u[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) {
      if (s < S) {
        const float4 v = *reinterpret_cast<const float4*>(x + (size_t)s * W + i);
        u[0] += coef[s] * v.x; u[1] += coef[s] * v.y; u[2] += coef[s] * v.z; u[3] += coef[s] * v.w;
      }
    }
    *reinterpret_cast<float4*>(u_s + i) = make_float4(u[0], u[1], u[2], u[3]);
    ss += u[0] * u[0] + u[1] * u[1] + u[2] * u[2] + u[3] * u[3];
  }
  ss = block_sum<kRowThreads>(ss, red);
  const float r = rsqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x * 4; i < W; i += kRowThreads * 4) {
    const float4 u = *reinterpret_cast<const float4*>(u_s + i);
    const float4 ww = *reinterpret_cast<const float4*>(w + i);
    const float n[4] = {u.x * r * (offset + ww.x), u.y * r * (offset + ww.y), u.z * r * (offset + ww.z),
                        u.w * r * (offset + ww.w)};
    store4<T>(out + (size_t)row * W + i, n);
    if (out32) store4<float>(out32 + (size_t)row * W + i, n);
  }
}

// grid (rows, column chunks of 512)
template <typename T>
__global__ void __launch_bounds__(128)
token_shift_vec_kernel(T* __restrict__ out, const float* __restrict__ n32, const float* __restrict__ mu,
                       float* __restrict__ state, const int* __restrict__ q_cu,
                       const int* __restrict__ positions, const int* __restrict__ token_seq,
                       const int* __restrict__ state_slots, int W) {
  const int row = blockIdx.x, i = (blockIdx.y * 128 + threadIdx.x) * 4;
  if (i >= W) return;
  const int seq = token_seq[row];
  const int first = q_cu[seq], last = q_cu[seq + 1] - 1;
  float n[4], p[4], m[4];
  load4<float>(n32 + (size_t)row * W + i, n);
  load4<float>(mu + i, m);
  if (row != first) {
    load4<float>(n32 + (size_t)(row - 1) * W + i, p);
  } else {
    float* slot = state + (size_t)state_slots[seq] * W + i;
    if (positions[row] == 0) { p[0] = p[1] = p[2] = p[3] = 0.0f; } else { load4<float>(slot, p); }
    float tail[4];
    load4<float>(n32 + (size_t)last * W + i, tail);
    store4<float>(slot, tail);
  }
  const float o[4] = {n[0] + (p[0] - n[0]) * m[0], n[1] + (p[1] - n[1]) * m[1], n[2] + (p[2] - n[2]) * m[2],
                      n[3] + (p[3] - n[3]) * m[3]};
  store4<T>(out + (size_t)row * W + i, o);
}

// grid (rows, column chunks of 512)
template <typename T>
__global__ void __launch_bounds__(128)
gated_hc_update_vec_kernel(float* __restrict__ X, const T* __restrict__ y, const T* __restrict__ gate,
                           const float* __restrict__ gate_bias, const float* __restrict__ mix,
                           const float* __restrict__ outc, int W, int S, int64_t ldy, int64_t ldg) {
  const int row = blockIdx.x, i = (blockIdx.y * 128 + threadIdx.x) * 4;
  if (i >= W) return;
  float* x = X + (size_t)row * S * W + i;
  float v[4];
  load4<T>(y + (size_t)row * ldy + i, v);
  if (gate) {
    float z[4], b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    load4<T>(gate + (size_t)row * ldg + i, z);
    if (gate_bias) load4<float>(gate_bias + i, b);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] *= 1.0f / (1.0f + expf(-(z[k] + b[k])));
  }
  float old[kMaxStreams][4];
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s)
    if (s < S) load4<float>(x + (size_t)s * W, old[s]);
#pragma unroll
  for (int t = 0; t < kMaxStreams; ++t) {
    if (t < S) {
      const float bt = outc ? outc[t] : 1.0f;
      float acc[4] = {bt * v[0], bt * v[1], bt * v[2], bt * v[3]};
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s) {
        if (s < S) {
          const float m = mix ? mix[s * S + t] : (s == t ? 1.0f : 0.0f);
#pragma unroll
          for (int k = 0; k < 4; ++k) acc[k] += m * old[s][k];
        }
      }
      store4<float>(x + (size_t)t * W, acc);
    }
  }
}

// out = act(in[:, :n]) * in[:, n:2n]; act 0 = SiLU, 1 = GELU (tanh form, tanhf), one rounding
template <typename T>
__global__ void gated_act_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int n,
                                 int64_t ld_in, int act) {
  const int64_t total = rows * n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n;
    const int c = (int)(idx - r * n);
    const float g = Num<T>::to_f(in[r * ld_in + c]);
    const float u = Num<T>::to_f(in[r * ld_in + n + c]);
    float a;
    if (act == 0) {
      a = g / (1.0f + expf(-g));
    } else {
      a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    }
    out[idx] = Num<T>::from_f(a * u);
  }
}

// out[t, h * d + i] = in[h, t, i] (* sigmoid(gate[t, h * d + i])): head-major rows back to token rows
template <typename T>
__global__ void heads_to_rows_kernel(T* __restrict__ out, const T* __restrict__ in,
                                     const T* __restrict__ gate, int64_t rows, int H, int d,
                                     int64_t ldg) {
  const int64_t total = rows * H * d;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / ((int64_t)H * d);
    const int rem = (int)(idx - t * H * d);
    const int h = rem / d, i = rem - h * d;
    float v = Num<T>::to_f(in[((int64_t)h * rows + t) * d + i]);
    if (gate) v *= 1.0f / (1.0f + expf(-Num<T>::to_f(gate[t * ldg + rem])));
    out[idx] = Num<T>::from_f(v);
  }
}

#define HYPER_DISPATCH(dtype, ...)                                               \
  switch (dtype) {                                                               \
    case B200_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }             \
    case B200_FP16: { using T = __half; __VA_ARGS__; break; }                    \
    case B200_FP32: { using T = float; __VA_ARGS__; break; }                     \
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);      \
  }

inline int ew_grid(int64_t total) {
  int64_t g = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_embed_streams(float* X, const void* table, const int32_t* tokens, int64_t rows, int64_t W,
                       int64_t S, int64_t vocab, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(X && table && tokens, "embed_streams: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && S >= 1 && S <= kMaxStreams && vocab > 0, "embed_streams: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  HYPER_DISPATCH(dtype, (embed_streams_kernel<T><<<(unsigned)rows, 128, 0, st>>>(
                            X, static_cast<const T*>(table), tokens, (int)W, (int)S, (int)vocab)));
  B200_LAUNCH_OK("embed_streams_kernel");
  return B200_OK;
}

int b200_hc_norm(void* out, float* out32, const float* X, const float* collapse, const float* weight,
                 int64_t rows, int64_t W, int64_t S, float eps, float offset, int dtype,
                 b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && X && weight, "hc_norm: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && W <= 12000 && S >= 1 && S <= kMaxStreams, "hc_norm: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  if (W % 4 == 0 && is_aligned(out, 16) && is_aligned(X, 16) && is_aligned(weight, 16) && (!out32 || is_aligned(out32, 16))) {
    HYPER_DISPATCH(dtype, (hc_norm_vec_kernel<T><<<(unsigned)rows, kRowThreads, W * sizeof(float), st>>>(
                              static_cast<T*>(out), out32, X, collapse, weight, (int)W, (int)S, eps, offset)));
    B200_LAUNCH_OK("hc_norm_vec_kernel");
    return B200_OK;
  }
  HYPER_DISPATCH(dtype, (hc_norm_kernel<T><<<(unsigned)rows, kRowThreads, W * sizeof(float), st>>>(
                            static_cast<T*>(out), out32, X, collapse, weight, (int)W, (int)S, eps, offset)));
  B200_LAUNCH_OK("hc_norm_kernel");
  return B200_OK;
}

int b200_token_shift(void* out, const float* n32, const float* mu, float* state, const int32_t* q_cu,
                     const int32_t* positions, const int32_t* token_seq, const int32_t* state_slots,
                     int64_t rows, int64_t W, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && n32 && mu && state && q_cu && positions && token_seq && state_slots,
                 "token_shift: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0, "token_shift: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  if (W % 4 == 0 && is_aligned(out, 16) && is_aligned(n32, 16) && is_aligned(mu, 16) && is_aligned(state, 16)) {
    dim3 grid((unsigned)rows, (unsigned)((W + 511) / 512));
    HYPER_DISPATCH(dtype, (token_shift_vec_kernel<T><<<grid, 128, 0, st>>>(
                              static_cast<T*>(out), n32, mu, state, q_cu, positions, token_seq, state_slots, (int)W)));
    B200_LAUNCH_OK("token_shift_vec_kernel");
    return B200_OK;
  }
  HYPER_DISPATCH(dtype, (token_shift_kernel<T><<<(unsigned)rows, 128, 0, st>>>(
                            static_cast<T*>(out), n32, mu, state, q_cu, positions, token_seq,
                            state_slots, (int)W)));
  B200_LAUNCH_OK("token_shift_kernel");
  return B200_OK;
}

int b200_gated_hc_update(float* X, const void* y, int64_t ldy, const void* gate, int64_t ldg,
                         const float* gate_bias, const float* mix, const float* outc, int64_t rows,
                         int64_t W, int64_t S, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(X && y, "gated_hc_update: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && S >= 1 && S <= kMaxStreams && ldy >= W && (!gate || ldg >= W),
                 "gated_hc_update: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  const int esz = dtype == B200_FP32 ? 4 : 2;
  if (W % 4 == 0 && is_aligned(X, 16) && is_aligned(y, 4 * esz) && (ldy * esz) % (4 * esz) == 0 &&
      (!gate || (is_aligned(gate, 4 * esz) && (ldg * esz) % (4 * esz) == 0)) && (!gate_bias || is_aligned(gate_bias, 16))) {
    dim3 grid((unsigned)rows, (unsigned)((W + 511) / 512));
    HYPER_DISPATCH(dtype, (gated_hc_update_vec_kernel<T><<<grid, 128, 0, st>>>(
                              X, static_cast<const T*>(y), static_cast<const T*>(gate), gate_bias, mix, outc, (int)W,
                              (int)S, ldy, ldg)));
    B200_LAUNCH_OK("gated_hc_update_vec_kernel");
    return B200_OK;
  }
  HYPER_DISPATCH(dtype, (gated_hc_update_kernel<T><<<(unsigned)rows, 128, 0, st>>>(
                            X, static_cast<const T*>(y), static_cast<const T*>(gate), gate_bias, mix,
                            outc, (int)W, (int)S, ldy, ldg)));
  B200_LAUNCH_OK("gated_hc_update_kernel");
  return B200_OK;
}

int b200_gated_act(void* out, const void* in, int64_t rows, int64_t n, int64_t ld_in, int act, int dtype,
                   b200_stream_t stream) {
  if (rows == 0 || n == 0) return B200_OK;
  B200_CHECK_ARG(out && in, "gated_act: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && n < (1ll << 30) && ld_in >= 2 * n && (act == 0 || act == 1),
                 "gated_act: bad shape / act (0 = silu, 1 = gelu tanh)");
  auto st = static_cast<cudaStream_t>(stream);
  HYPER_DISPATCH(dtype, (gated_act_kernel<T><<<ew_grid(rows * n), 256, 0, st>>>(
                            static_cast<T*>(out), static_cast<const T*>(in), rows, (int)n, ld_in, act)));
  B200_LAUNCH_OK("gated_act_kernel");
  return B200_OK;
}

int b200_heads_to_rows(void* out, const void* in, const void* gate, int64_t ldg, int64_t rows, int64_t H,
                       int64_t d, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && in, "heads_to_rows: null pointer");
  B200_CHECK_ARG(rows > 0 && H > 0 && d > 0 && H * d < (1ll << 30) && (!gate || ldg >= H * d),
                 "heads_to_rows: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  HYPER_DISPATCH(dtype, (heads_to_rows_kernel<T><<<ew_grid(rows * H * d), 256, 0, st>>>(
                            static_cast<T*>(out), static_cast<const T*>(in), static_cast<const T*>(gate),
                            rows, (int)H, (int)d, ldg)));
  B200_LAUNCH_OK("heads_to_rows_kernel");
  return B200_OK;
}

}  // extern "C"
