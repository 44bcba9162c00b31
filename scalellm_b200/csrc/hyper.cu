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
