// delta_rule.cu — generalised delta-rule recurrence with a per-channel decay and removal rate.
//
// Per head, state S [d (key) x d (value)] in fp32, carried per sequence in a state slot:
//     w_t = exp(-decay_scale * sigmoid(wl_t + w0))        decay per key channel
//     a_t = sigmoid(al_t + a0)                            removal rate per key channel
//     u_t = k_t / sqrt(|k_t|^2 + key_eps)                 unit key
//     S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T
//     o_t = S_t^T r_t
//     out = o_t / rms(o_t) * nw * sigmoid(g_t)            per-head RMS, channel weight, output gate
// One CTA per (sequence, head); thread j owns column j of S in registers and walks the step's
// tokens of that sequence in order (a single decoded token or a whole prompt portion).  A portion
// that starts at position 0 starts from S = 0 instead of reading the slot.
#include "common.cuh"

namespace b200 {
namespace {

template <typename T, int DK>
__global__ void __launch_bounds__(DK < 32 ? 32 : DK)
delta_rule_kernel(T* __restrict__ out, int64_t ldo, const T* __restrict__ r, const T* __restrict__ k,
                  const T* __restrict__ v, const T* __restrict__ wl, const T* __restrict__ al,
                  const T* __restrict__ g, int64_t ld, int64_t ld_w, const float* __restrict__ w0,
                  const float* __restrict__ a0, const float* __restrict__ nw, float* __restrict__ state,
                  const int* __restrict__ q_cu, const int* __restrict__ positions,
                  const int* __restrict__ state_slots, int H, int d, float decay_scale, float key_eps,
                  float eps) {
  constexpr int NT = DK < 32 ? 32 : DK;
  __shared__ __align__(16) float r_s[DK], k_s[DK], u_s[DK], w_s[DK], au_s[DK];
  __shared__ float red[32], red2[32];   // alternate: block_sum does not sync after reading
  const int seq = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int t0 = q_cu[seq], t1 = q_cu[seq + 1];
  if (t0 >= t1) return;
  const bool live = j < d;
  if (j < DK && !live) r_s[j] = k_s[j] = u_s[j] = w_s[j] = au_s[j] = 0.0f;   // padding entries stay zero
  float* Sg = state + (((size_t)state_slots[seq] * H + h) * d) * d;   // [key][value]
  float S[DK];
  const bool fresh = positions[t0] == 0;
#pragma unroll
  for (int kk = 0; kk < DK; ++kk) S[kk] = (live && kk < d && !fresh) ? Sg[(size_t)kk * d + j] : 0.0f;
  const int c = h * d + j;
  const float w0j = live ? w0[c] : 0.0f, a0j = live ? a0[c] : 0.0f, nwj = live ? nw[c] : 0.0f;
  // the six inputs of token t + 1 are loaded while token t is computed: the recurrence itself is short,
  // a dependent global load per token would dominate it
  float nk = 0.0f, nv = 0.0f, nr = 0.0f, nwl = 0.0f, nal = 0.0f, ng = 0.0f;
  auto load_token = [&](int t) {
    if (live) {
      const size_t base = (size_t)t * ld + c;
      nk = Num<T>::to_f(k[base]);
      nv = Num<T>::to_f(v[base]);
      nr = Num<T>::to_f(r[base]);
      nal = Num<T>::to_f(al[base]);
      ng = Num<T>::to_f(g[base]);
      nwl = Num<T>::to_f(wl[(size_t)t * ld_w + c]);
    }
  };
  load_token(t0);
  for (int t = t0; t < t1; ++t) {
    const float kj = nk, vj = nv, alj = nal, gj = ng;
    if (live) {
      r_s[j] = nr;
      k_s[j] = kj;
      const float sw = 1.0f / (1.0f + expf(-(nwl + w0j)));
      w_s[j] = expf(-decay_scale * sw);
    }
    if (t + 1 < t1) load_token(t + 1);
    const float k2 = block_sum<NT>(kj * kj, red);   // syncs: the vectors above are visible after it
    if (live) {
      const float uj = kj * rsqrtf(k2 + key_eps);
      const float aj = 1.0f / (1.0f + expf(-(alj + a0j)));
      u_s[j] = uj;
      au_s[j] = aj * uj;
    }
    __syncthreads();
    // both passes over the key dimension read the shared vectors four at a time and keep four partial sums, so
    // that neither the shared-memory loads nor one long chain of dependent FMAs set the pace (entries >= d are 0)
    float us4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int kk = 0; kk < DK; kk += 4) {
      const float4 u4 = *reinterpret_cast<const float4*>(u_s + kk);
      us4[0] += u4.x * S[kk]; us4[1] += u4.y * S[kk + 1]; us4[2] += u4.z * S[kk + 2]; us4[3] += u4.w * S[kk + 3];
    }
    const float uS = (us4[0] + us4[1]) + (us4[2] + us4[3]);
    float o4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int kk = 0; kk < DK; kk += 4) {
      const float4 w4 = *reinterpret_cast<const float4*>(w_s + kk);
      const float4 a4 = *reinterpret_cast<const float4*>(au_s + kk);
      const float4 k4 = *reinterpret_cast<const float4*>(k_s + kk);
      const float4 r4 = *reinterpret_cast<const float4*>(r_s + kk);
      S[kk] = w4.x * S[kk] - a4.x * uS + k4.x * vj;             o4[0] += S[kk] * r4.x;
      S[kk + 1] = w4.y * S[kk + 1] - a4.y * uS + k4.y * vj;     o4[1] += S[kk + 1] * r4.y;
      S[kk + 2] = w4.z * S[kk + 2] - a4.z * uS + k4.z * vj;     o4[2] += S[kk + 2] * r4.z;
      S[kk + 3] = w4.w * S[kk + 3] - a4.w * uS + k4.w * vj;     o4[3] += S[kk + 3] * r4.w;
    }
    const float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
    const float o2 = block_sum<NT>(live ? o * o : 0.0f, red2);   // also fences the smem vectors
    if (live) {
      const float gate = 1.0f / (1.0f + expf(-gj));
      out[(size_t)t * ldo + c] = Num<T>::from_f(o * rsqrtf(o2 / (float)d + eps) * nwj * gate);
    }
  }
  if (live) {
#pragma unroll
    for (int kk = 0; kk < DK; ++kk)
      if (kk < d) Sg[(size_t)kk * d + j] = S[kk];
  }
}

template <typename T>
int launch_delta(void* out, int64_t ldo, const void* r, const void* k, const void* v, const void* wl,
                 const void* al, const void* g, int64_t ld, int64_t ld_w, const float* w0, const float* a0,
                 const float* nw, float* state, const int* q_cu, const int* positions,
                 const int* state_slots, int64_t n_seq, int H, int d, float decay_scale, float key_eps,
                 float eps, cudaStream_t st) {
  dim3 grid((unsigned)n_seq, (unsigned)H);
#define DR_LAUNCH(DK)                                                                                 \
  delta_rule_kernel<T, DK><<<grid, (DK < 32 ? 32 : DK), 0, st>>>(                                      \
      static_cast<T*>(out), ldo, static_cast<const T*>(r), static_cast<const T*>(k),                   \
      static_cast<const T*>(v), static_cast<const T*>(wl), static_cast<const T*>(al),                  \
      static_cast<const T*>(g), ld, ld_w, w0, a0, nw, state, q_cu, positions, state_slots, H, d, decay_scale, \
      key_eps, eps)
  if (d <= 32) DR_LAUNCH(32);
  else if (d <= 64) DR_LAUNCH(64);
  else if (d <= 128) DR_LAUNCH(128);
  else return set_error(B200_ERR_UNSUPPORTED, "delta_rule: head size %d > 128", d);
#undef DR_LAUNCH
  B200_LAUNCH_OK("delta_rule_kernel");
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_delta_rule(void* out, int64_t ldo, const void* r, const void* k, const void* v,
                    const void* decay_logits, const void* removal_logits, const void* gate_logits,
                    int64_t ld, int64_t ld_decay, const float* decay_bias, const float* removal_bias,
                    const float* norm_weight, float* state, const int32_t* q_cu_lens,
                    const int32_t* positions, const int32_t* state_slots, int64_t n_seq, int64_t H,
                    int64_t d, float decay_scale, float key_eps, float eps, int dtype,
                    b200_stream_t stream) {
  if (n_seq == 0) return B200_OK;
  B200_CHECK_ARG(out && r && k && v && decay_logits && removal_logits && gate_logits && decay_bias &&
                     removal_bias && norm_weight && state && q_cu_lens && positions && state_slots,
                 "delta_rule: null pointer");
  B200_CHECK_ARG(n_seq > 0 && H > 0 && H <= 65535 && d > 0 && ldo >= H * d && ld >= H * d && ld_decay >= H * d, "delta_rule: bad shape");
  auto st = static_cast<cudaStream_t>(stream);
#define DR_CALL(T)                                                                                      \
  return launch_delta<T>(out, ldo, r, k, v, decay_logits, removal_logits, gate_logits, ld, ld_decay, decay_bias,  \
                         removal_bias, norm_weight, state, q_cu_lens, positions, state_slots, n_seq,    \
                         (int)H, (int)d, decay_scale, key_eps, eps, st)
  switch (dtype) {
    case B200_BF16: DR_CALL(__nv_bfloat16);
    case B200_FP16: DR_CALL(__half);
    case B200_FP32: DR_CALL(float);
    default: return set_error(B200_ERR_INVALID_ARG, "bad dtype %d", dtype);
  }
#undef DR_CALL
}

}  // extern "C"
