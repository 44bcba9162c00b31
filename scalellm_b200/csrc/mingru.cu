// mingru.cu — minimal gated recurrent unit: a per-channel linear recurrence whose gate and candidate
// depend on the current token only.
//
//     z_t = sigmoid(pz_t + bz)                         update gate
//     u_t = px_t + bx ;  c_t = u_t + 1/2 (u_t >= 0) | sigmoid(u_t) (u_t < 0)     positive candidate
//     S_t = (1 - z_t) S_{t-1} + z_t c_t                state, fp32, one value per channel
//     out_t = S_t * silu(pg_t)
//
// pz | px | pg are the three column blocks [width] of one projection matrix (row stride ld).  The state of a
// sequence lives in its state slot [n_slots, width]; a portion whose first row has position 0 starts from 0.
// One thread per (sequence, channel) walks the step's tokens of that sequence in order; the three inputs of the
// following tokens are loaded ahead, since nothing of them depends on the recurrence.
// Long portions are cut into chunks of `chunk_len` tokens that run side by side: the recurrence is linear in S
// (S_t = a_t S_{t-1} + b_t with a = 1 - z, b = z c), so a first kernel reduces every chunk to (A, B) with
// S_end = A S_start + B, and a second one starts every chunk from the fold of the chunks before it.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kAhead = 4;

template <typename T>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(T* __restrict__ out, int64_t ldo, const T* __restrict__ proj, int64_t ld,
                   const float* __restrict__ z_bias, const float* __restrict__ x_bias, float* __restrict__ state,
                   const int* __restrict__ q_cu, const int* __restrict__ positions,
                   const int* __restrict__ state_slots, int width) {
  const int seq = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int t0 = q_cu[seq], t1 = q_cu[seq + 1];
  if (c >= width || t0 >= t1) return;
  float* slot = state + (size_t)state_slots[seq] * width + c;
  float S = positions[t0] == 0 ? 0.0f : *slot;
  const float bz = z_bias ? z_bias[c] : 0.0f, bx = x_bias ? x_bias[c] : 0.0f;
  float pz[kAhead], px[kAhead], pg[kAhead];
  auto load = [&](int t, int k) {
    const T* p = proj + (size_t)t * ld + c;
    pz[k] = Num<T>::to_f(p[0]);
    px[k] = Num<T>::to_f(p[width]);
    pg[k] = Num<T>::to_f(p[2 * (size_t)width]);
  };
#pragma unroll
  for (int k = 0; k < kAhead; ++k)
    if (t0 + k < t1) load(t0 + k, k);
  for (int t = t0; t < t1; t += kAhead) {
    float cz[kAhead], cx[kAhead], cg[kAhead];
#pragma unroll
    for (int k = 0; k < kAhead; ++k) { cz[k] = pz[k]; cx[k] = px[k]; cg[k] = pg[k]; }
#pragma unroll
    for (int k = 0; k < kAhead; ++k)
      if (t + kAhead + k < t1) load(t + kAhead + k, k);
#pragma unroll
    for (int k = 0; k < kAhead; ++k) {
      if (t + k < t1) {
        const float z = 1.0f / (1.0f + expf(-(cz[k] + bz)));
        const float u = cx[k] + bx;
        const float cand = u >= 0.0f ? u + 0.5f : 1.0f / (1.0f + expf(-u));
        S = (1.0f - z) * S + z * cand;
        const float g = cg[k];
        out[(size_t)(t + k) * ldo + c] = Num<T>::from_f(S * (g / (1.0f + expf(-g))));
      }
    }
  }
  *slot = S;
}

// (A, B) of every chunk, and the state every sequence starts from (its slot, or 0 at position 0)
template <typename T>
__global__ void __launch_bounds__(128)
mingru_chunk_summary_kernel(float* __restrict__ A_ws, float* __restrict__ B_ws, float* __restrict__ S0_ws,
                            const T* __restrict__ proj, int64_t ld, const float* __restrict__ z_bias,
                            const float* __restrict__ x_bias, const float* __restrict__ state,
                            const int* __restrict__ q_cu, const int* __restrict__ positions,
                            const int* __restrict__ state_slots, int width, int chunk_len, int n_chunks) {
  const int seq = blockIdx.x, chunk = blockIdx.y;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  const int q0 = q_cu[seq], q1 = q_cu[seq + 1];
  const int t0 = q0 + chunk * chunk_len;
  if (c >= width || t0 >= q1) return;
  const int t1 = t0 + chunk_len < q1 ? t0 + chunk_len : q1;
  if (chunk == 0)
    S0_ws[(size_t)seq * width + c] = positions[q0] == 0 ? 0.0f : state[(size_t)state_slots[seq] * width + c];
  if (t1 == q1) return;                       // nothing follows the portion's last chunk
  const float bz = z_bias ? z_bias[c] : 0.0f, bx = x_bias ? x_bias[c] : 0.0f;
  float A = 1.0f, B = 0.0f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const T* p = proj + (size_t)t * ld + c;
    const float z = 1.0f / (1.0f + expf(-(Num<T>::to_f(p[0]) + bz)));
    const float u = Num<T>::to_f(p[width]) + bx;
    const float cand = u >= 0.0f ? u + 0.5f : 1.0f / (1.0f + expf(-u));
    A *= 1.0f - z;
    B = (1.0f - z) * B + z * cand;
  }
  const size_t o = ((size_t)seq * n_chunks + chunk) * width + c;
  A_ws[o] = A;
  B_ws[o] = B;
}

template <typename T>
__global__ void __launch_bounds__(128)
mingru_chunk_apply_kernel(T* __restrict__ out, int64_t ldo, const T* __restrict__ proj, int64_t ld,
                          const float* __restrict__ z_bias, const float* __restrict__ x_bias,
                          float* __restrict__ state, const float* __restrict__ A_ws, const float* __restrict__ B_ws,
                          const float* __restrict__ S0_ws, const int* __restrict__ q_cu,
                          const int* __restrict__ state_slots, int width, int chunk_len, int n_chunks) {
  const int seq = blockIdx.x, chunk = blockIdx.y;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  const int q0 = q_cu[seq], q1 = q_cu[seq + 1];
  const int t0 = q0 + chunk * chunk_len;
  if (c >= width || t0 >= q1) return;
  const int t1 = t0 + chunk_len < q1 ? t0 + chunk_len : q1;
  float S = S0_ws[(size_t)seq * width + c];
  for (int k = 0; k < chunk; ++k) {
    const size_t o = ((size_t)seq * n_chunks + k) * width + c;
    S = A_ws[o] * S + B_ws[o];
  }
  const float bz = z_bias ? z_bias[c] : 0.0f, bx = x_bias ? x_bias[c] : 0.0f;
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const T* p = proj + (size_t)t * ld + c;
    const float z = 1.0f / (1.0f + expf(-(Num<T>::to_f(p[0]) + bz)));
    const float u = Num<T>::to_f(p[width]) + bx;
    const float cand = u >= 0.0f ? u + 0.5f : 1.0f / (1.0f + expf(-u));
    S = (1.0f - z) * S + z * cand;
    const float g = Num<T>::to_f(p[2 * (size_t)width]);
    out[(size_t)t * ldo + c] = Num<T>::from_f(S * (g / (1.0f + expf(-g))));
  }
  if (t1 == q1) state[(size_t)state_slots[seq] * width + c] = S;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_mingru_scan(void* out, int64_t ldo, const void* proj, int64_t ld, const float* z_bias,
                     const float* x_bias, float* state, const int32_t* q_cu_lens, const int32_t* positions,
                     const int32_t* state_slots, int64_t n_seq, int64_t width, int dtype, b200_stream_t stream) {
  if (n_seq == 0) return B200_OK;
  B200_CHECK_ARG(out && proj && state && q_cu_lens && positions && state_slots, "mingru_scan: null pointer");
  B200_CHECK_ARG(n_seq > 0 && width > 0 && width < (1ll << 24) && ldo >= width && ld >= 3 * width,
                 "mingru_scan: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)n_seq, (unsigned)((width + 127) / 128));
#define MG_CALL(T)                                                                                          \
  mingru_scan_kernel<T><<<grid, 128, 0, st>>>(static_cast<T*>(out), ldo, static_cast<const T*>(proj), ld,   \
                                              z_bias, x_bias, state, q_cu_lens, positions, state_slots, (int)width)
  switch (dtype) {
    case B200_BF16: MG_CALL(__nv_bfloat16); break;
    case B200_FP16: MG_CALL(__half); break;
    case B200_FP32: MG_CALL(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef MG_CALL
  B200_LAUNCH_OK("mingru_scan_kernel");
  return B200_OK;
}

int64_t b200_mingru_chunked_workspace_floats(int64_t n_seq, int64_t width, int64_t q_max, int64_t chunk_len) {
  if (n_seq <= 0 || width <= 0 || q_max <= 0 || chunk_len <= 0) return 0;
  const int64_t n_chunks = (q_max + chunk_len - 1) / chunk_len;
  return n_seq * (2 * n_chunks + 1) * width;
}

int b200_mingru_scan_chunked(void* out, int64_t ldo, const void* proj, int64_t ld, const float* z_bias,
                             const float* x_bias, float* state, const int32_t* q_cu_lens, const int32_t* positions,
                             const int32_t* state_slots, int64_t n_seq, int64_t width, int64_t q_max,
                             int64_t chunk_len, float* workspace, int64_t workspace_floats, int dtype,
                             b200_stream_t stream) {
  if (n_seq == 0 || q_max == 0) return B200_OK;
  B200_CHECK_ARG(out && proj && state && q_cu_lens && positions && state_slots && workspace,
                 "mingru_scan_chunked: null pointer");
  B200_CHECK_ARG(n_seq > 0 && width > 0 && width < (1ll << 24) && ldo >= width && ld >= 3 * width && q_max > 0 &&
                     chunk_len > 0, "mingru_scan_chunked: bad shape");
  const int64_t n_chunks = (q_max + chunk_len - 1) / chunk_len;
  B200_CHECK_ARG(n_chunks <= 65535 && (width + 127) / 128 <= 65535 &&
                     workspace_floats >= b200_mingru_chunked_workspace_floats(n_seq, width, q_max, chunk_len),
                 "mingru_scan_chunked: too many chunks or a workspace too small");
  auto st = static_cast<cudaStream_t>(stream);
  float* A_ws = workspace;
  float* B_ws = A_ws + n_seq * n_chunks * width;
  float* S0_ws = B_ws + n_seq * n_chunks * width;
  dim3 grid((unsigned)n_seq, (unsigned)n_chunks, (unsigned)((width + 127) / 128));
#define MGC_CALL(T)                                                                                              \
  do {                                                                                                           \
    mingru_chunk_summary_kernel<T><<<grid, 128, 0, st>>>(A_ws, B_ws, S0_ws, static_cast<const T*>(proj), ld,     \
                                                         z_bias, x_bias, state, q_cu_lens, positions,            \
                                                         state_slots, (int)width, (int)chunk_len, (int)n_chunks); \
    mingru_chunk_apply_kernel<T><<<grid, 128, 0, st>>>(static_cast<T*>(out), ldo, static_cast<const T*>(proj),   \
                                                       ld, z_bias, x_bias, state, A_ws, B_ws, S0_ws, q_cu_lens,  \
                                                       state_slots, (int)width, (int)chunk_len, (int)n_chunks);  \
  } while (0)
  switch (dtype) {
    case B200_BF16: MGC_CALL(__nv_bfloat16); break;
    case B200_FP16: MGC_CALL(__half); break;
    case B200_FP32: MGC_CALL(float); break;
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef MGC_CALL
  B200_LAUNCH_OK("mingru_chunk kernels");
  return B200_OK;
}

}  // extern "C"
