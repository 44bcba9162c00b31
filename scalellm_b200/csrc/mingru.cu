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

}  // extern "C"
