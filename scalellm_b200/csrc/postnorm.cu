// postnorm.cu — kernels for decoders that normalise a sublayer's RESULT (not its input) before it
// enters an fp32 residual, and that feed every layer a learned average of all earlier layers' results.
//
//   embed     x = scale * E[tok] + B[(mul_prev * prev + mul_cur * tok) mod buckets]   (B[buckets] when a
//             sequence starts: prev < 0); the hashed pair table B is optional
//   postnorm  r = x + mult * y / sqrt(mean_g(y^2) + eps) * w     mean over the channel's group: the row is cut
//             into `groups` equal consecutive parts, each with its own root mean square
//   history   H[n - 1] = r ; x' = sum_{j < n} c[j] H[j]          (optional) the depth-weighted average
//   glu       out = g sigmoid(slope g) (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit)
//   token gate out = gelu_tanh(a) * table[tok, col0 + c]          a per-token learned vector gates a projection
//
// The residual, the history, sums of squares and every transcendental are fp32; T is the activation type
// of y and of the copy of the residual that the next matrix product reads.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kRowThreads = 256;

template <typename T>
__global__ void bigram_embed_kernel(float* __restrict__ x, T* __restrict__ h, const T* __restrict__ table,
                                    const T* __restrict__ pair_table, const int* __restrict__ tokens,
                                    const int* __restrict__ prev_tokens, int W, int vocab, int64_t buckets,
                                    int64_t mul_prev, int64_t mul_cur, float scale) {
  const int row = blockIdx.x;
  int tok = tokens[row];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const T* src = table + (size_t)tok * W;
  const T* pair = nullptr;
  if (pair_table) {
    const int prev = prev_tokens ? prev_tokens[row] : -1;
    const int64_t r = prev < 0 ? buckets : ((int64_t)prev * mul_prev + (int64_t)tok * mul_cur) % buckets;
    pair = pair_table + (size_t)r * W;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = Num<T>::to_f(src[i]) * scale;
    if (pair) v += Num<T>::to_f(pair[i]);
    x[(size_t)row * W + i] = v;
    if (h) h[(size_t)row * W + i] = Num<T>::from_f(v);
  }
}

// one CTA per row; y is held in shared memory between the two passes; warp w owns groups w, w + 8, ...
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
postnorm_residual_kernel(float* __restrict__ x_out, T* __restrict__ h_out, const float* __restrict__ x_in,
                         const T* __restrict__ y, int64_t ldy, const float* __restrict__ w, int W, int groups,
                         float mult, float eps, float* __restrict__ hist, int64_t hist_stride, int n_hist,
                         const float* __restrict__ coef) {
  extern __shared__ float sm[];
  float* y_s = sm;            // [W]
  float* r_s = sm + W;        // [groups] reciprocal root mean squares
  const int row = blockIdx.x;
  const int gs = W / groups;
  for (int i = threadIdx.x; i < W; i += kRowThreads) y_s[i] = Num<T>::to_f(y[(size_t)row * ldy + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < groups; g += kRowThreads / 32) {
    float ss = 0.0f;
    for (int i = lane; i < gs; i += 32) {
      const float v = y_s[g * gs + i];
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) r_s[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  const size_t base = (size_t)row * W;
  for (int i = threadIdx.x; i < W; i += kRowThreads) {
    float r = x_in[base + i] + mult * (y_s[i] * r_s[i / gs] * w[i]);
    if (hist) {
      hist[(size_t)(n_hist - 1) * hist_stride + base + i] = r;
      float acc = coef[n_hist - 1] * r;
      for (int j = n_hist - 2; j >= 0; --j) acc += coef[j] * hist[(size_t)j * hist_stride + base + i];
      r = acc;
    }
    x_out[base + i] = r;
    if (h_out) h_out[base + i] = Num<T>::from_f(r);
  }
}

// out = x / sqrt(mean_group(x^2) + eps) * w for fp32 rows x, written as T; one CTA per row
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
group_rms_norm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, int W,
                      int groups, float eps) {
  extern __shared__ float sm[];
  float* x_s = sm;
  float* r_s = sm + W;
  const int row = blockIdx.x;
  const int gs = W / groups;
  for (int i = threadIdx.x; i < W; i += kRowThreads) x_s[i] = x[(size_t)row * W + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < groups; g += kRowThreads / 32) {
    float ss = 0.0f;
    for (int i = lane; i < gs; i += 32) {
      const float v = x_s[g * gs + i];
      ss += v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) r_s[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += kRowThreads)
    out[(size_t)row * W + i] = Num<T>::from_f(x_s[i] * r_s[i / gs] * w[i]);
}

template <typename T>
__global__ void glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int n,
                                   int64_t ld_in, float limit, float slope) {
  const int64_t total = rows * n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n;
    const int c = (int)(idx - r * n);
    const float g = fminf(Num<T>::to_f(in[r * ld_in + c]), limit);
    const float u = fminf(fmaxf(Num<T>::to_f(in[r * ld_in + n + c]), -limit), limit);
    out[idx] = Num<T>::from_f(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
  }
}

template <typename T>
__global__ void token_gated_gelu_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t ld_in,
                                        const T* __restrict__ table, int64_t ld_table, int col0,
                                        const int* __restrict__ tokens, int64_t rows, int n, int vocab) {
  const int64_t total = rows * n;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n;
    const int c = (int)(idx - r * n);
    int tok = tokens[r];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const float a = Num<T>::to_f(in[r * ld_in + c]);
    const float e = Num<T>::to_f(table[(int64_t)tok * ld_table + col0 + c]);
    const float gl = 0.5f * a * (1.0f + tanhf(0.7978845608028654f * (a + 0.044715f * a * a * a)));
    out[idx] = Num<T>::from_f(gl * e);
  }
}

#define POSTNORM_DISPATCH(dtype, ...)                                            \
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

int b200_bigram_embed(float* x, void* h, const void* table, const void* pair_table, const int32_t* tokens,
                      const int32_t* prev_tokens, int64_t rows, int64_t W, int64_t vocab, int64_t buckets,
                      int64_t mul_prev, int64_t mul_cur, float scale, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x && table && tokens, "bigram_embed: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && vocab > 0 && W < (1ll << 30) && (!pair_table || buckets > 0),
                 "bigram_embed: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  POSTNORM_DISPATCH(dtype, (bigram_embed_kernel<T><<<(unsigned)rows, 256, 0, st>>>(
                               x, static_cast<T*>(h), static_cast<const T*>(table),
                               static_cast<const T*>(pair_table), tokens, prev_tokens, (int)W, (int)vocab,
                               buckets, mul_prev, mul_cur, scale)));
  B200_LAUNCH_OK("bigram_embed_kernel");
  return B200_OK;
}

int b200_postnorm_residual(float* x_out, void* h_out, const float* x_in, const void* y, int64_t ldy,
                           const float* weight, int64_t rows, int64_t W, int64_t groups, float mult, float eps,
                           float* hist, int64_t hist_stride, int64_t n_hist, const float* coef, int dtype,
                           b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(x_out && x_in && y && weight, "postnorm_residual: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && groups > 0 && W % groups == 0 && ldy >= W && (W + groups) * 4 <= 200 * 1024,
                 "postnorm_residual: bad shape (W a multiple of groups, at most ~50K channels)");
  B200_CHECK_ARG(!hist || (n_hist > 0 && coef && hist_stride >= rows * W), "postnorm_residual: bad history");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(W + groups) * sizeof(float);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(postnorm_residual_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    postnorm_residual_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(
        x_out, static_cast<T*>(h_out), x_in, static_cast<const T*>(y), ldy, weight, (int)W, (int)groups, mult,
        eps, hist, hist_stride, (int)n_hist, coef);
  });
  B200_LAUNCH_OK("postnorm_residual_kernel");
  return B200_OK;
}

int b200_group_rms_norm(void* out, const float* x, const float* weight, int64_t rows, int64_t W, int64_t groups,
                        float eps, int dtype, b200_stream_t stream) {
  if (rows == 0) return B200_OK;
  B200_CHECK_ARG(out && x && weight, "group_rms_norm: null pointer");
  B200_CHECK_ARG(rows > 0 && W > 0 && groups > 0 && W % groups == 0 && (W + groups) * 4 <= 200 * 1024,
                 "group_rms_norm: bad shape (W a multiple of groups, at most ~50K channels)");
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)(W + groups) * sizeof(float);
  POSTNORM_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(group_rms_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    group_rms_norm_kernel<T><<<(unsigned)rows, kRowThreads, smem, st>>>(static_cast<T*>(out), x, weight, (int)W,
                                                                        (int)groups, eps);
  });
  B200_LAUNCH_OK("group_rms_norm_kernel");
  return B200_OK;
}

int b200_glu_clamped(void* out, const void* in, int64_t rows, int64_t n, int64_t ld_in, float limit, float slope,
                     int dtype, b200_stream_t stream) {
  if (rows == 0 || n == 0) return B200_OK;
  B200_CHECK_ARG(out && in, "glu_clamped: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && n < (1ll << 30) && ld_in >= 2 * n, "glu_clamped: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  POSTNORM_DISPATCH(dtype, (glu_clamped_kernel<T><<<ew_grid(rows * n), 256, 0, st>>>(
                               static_cast<T*>(out), static_cast<const T*>(in), rows, (int)n, ld_in, limit, slope)));
  B200_LAUNCH_OK("glu_clamped_kernel");
  return B200_OK;
}

int b200_token_gated_gelu(void* out, const void* in, int64_t ld_in, const void* table, int64_t ld_table,
                          int64_t col0, const int32_t* tokens, int64_t rows, int64_t n, int64_t vocab, int dtype,
                          b200_stream_t stream) {
  if (rows == 0 || n == 0) return B200_OK;
  B200_CHECK_ARG(out && in && table && tokens, "token_gated_gelu: null pointer");
  B200_CHECK_ARG(rows > 0 && n > 0 && n < (1ll << 30) && ld_in >= n && col0 >= 0 && ld_table >= col0 + n && vocab > 0,
                 "token_gated_gelu: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  POSTNORM_DISPATCH(dtype, (token_gated_gelu_kernel<T><<<ew_grid(rows * n), 256, 0, st>>>(
                               static_cast<T*>(out), static_cast<const T*>(in), ld_in, static_cast<const T*>(table),
                               ld_table, (int)col0, tokens, rows, (int)n, (int)vocab)));
  B200_LAUNCH_OK("token_gated_gelu_kernel");
  return B200_OK;
}

}  // extern "C"
