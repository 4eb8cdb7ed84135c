// Gated delta rule with one decay per head and key channel, over packed tokens of several requests.
// A request's state lives in a slot: S [heads, D, Vd] in fp32 and the last (taps - 1) inputs of the
// short convolutions, fp32 as well.
//
//   delta_prepare_kernel     a block a token: causal convolution over time (taps from the rows of
//                            this step, or from the slot where the step's portion starts later than
//                            the tap reaches) + SiLU on the q | k | v channels; q and k made unit
//                            vectors per head (q also times D^-1/2); decay g = exp(-exp(A_log_h) *
//                            softplus(a + dt_bias)); beta = sigmoid(b).  Everything leaves in fp32.
//   delta_conv_state_kernel  a thread a (request, channel): the slot's last inputs after the step.
//   delta_recurrence_kernel  per (request, head): S <- g * S (rows); u = beta (v - S^T k);
//                            S <- S + k u^T; o = S^T q, token after token.  The columns of S are
//                            independent: four lanes share a column (a quarter of the rows each, in
//                            registers), a block holds 32 columns.  The next token's operands are
//                            loaded while the current one is worked on.
//   delta_output_kernel      a warp a (token, head): o / rms(o) * w * sigmoid(gate).
#include "common.cuh"

namespace gf {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

struct DeltaDims {
  int H, G, D, Vd, taps;
  int channels;          // 2 G D + H Vd: the convolved columns q | k | v of a projection row
  int state_stride;      // floats a slot
  int conv_off;          // where the convolution inputs start in a slot
};

template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, int ld, int b_off,
                                     const float* __restrict__ a, const float* __restrict__ conv_w,
                                     const float* __restrict__ dt_bias,
                                     const float* __restrict__ A_log,
                                     const float* __restrict__ state,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ cu_seqlens,
                                     const int* __restrict__ slot_ids, DeltaDims dm,
                                     float* __restrict__ qn, float* __restrict__ kn,
                                     float* __restrict__ v, float* __restrict__ g,
                                     float* __restrict__ beta) {
  extern __shared__ float y[];                    // the token's convolved channels
  const int r = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const int b = seq_of_token[r];
  const int i = r - cu_seqlens[b];                // place in this step's portion
  const float* cs = state + (size_t)slot_ids[b] * dm.state_stride + dm.conv_off;
  const int taps = dm.taps, CH = dm.channels;
  for (int ch = threadIdx.x; ch < CH; ch += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int off = i - (taps - 1 - j);         // place of the tap's input in the portion
      const float x = off >= 0 ? to_f32(proj[(size_t)(r - (taps - 1 - j)) * ld + ch])
                               : cs[(size_t)(taps - 1 + off) * CH + ch];
      acc = fmaf(conv_w[(size_t)ch * taps + j], x, acc);
    }
    y[ch] = acc * sigmoid_f(acc);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int GD = dm.G * dm.D;
  for (int u = warp; u < 2 * dm.G; u += nwarps) {  // unit vectors: q heads, then k heads
    const float* src = y + (size_t)u * dm.D;
    float ss = 0.f;
    for (int d = lane; d < dm.D; d += 32) ss += src[d] * src[d];
    ss = warp_sum(ss);
    const bool is_q = u < dm.G;
    const float f = (is_q ? rsqrtf((float)dm.D) : 1.f) / sqrtf(ss + 1e-6f);
    float* dst = (is_q ? qn : kn) + (size_t)r * GD + (size_t)(is_q ? u : u - dm.G) * dm.D;
    for (int d = lane; d < dm.D; d += 32) dst[d] = src[d] * f;
  }
  const int HV = dm.H * dm.Vd, HD = dm.H * dm.D;
  for (int j = threadIdx.x; j < HV; j += blockDim.x) v[(size_t)r * HV + j] = y[2 * GD + j];
  for (int j = threadIdx.x; j < HD; j += blockDim.x) {
    const float rate = expf(A_log[j / dm.D]);
    g[(size_t)r * HD + j] = expf(-rate * softplus_f(a[(size_t)r * HD + j] + dt_bias[j]));
  }
  for (int h = threadIdx.x; h < dm.H; h += blockDim.x)
    beta[(size_t)r * dm.H + h] = sigmoid_f(to_f32(proj[(size_t)r * ld + b_off + h]));
}

template <typename T>
__global__ void delta_conv_state_kernel(const T* __restrict__ proj, int ld,
                                        float* __restrict__ state,
                                        const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ slot_ids, DeltaDims dm) {
  const int b = blockIdx.y;
  const int ch = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_trigger();
  pdl_wait();
  if (ch >= dm.channels) return;
  const int start = cu_seqlens[b], n = cu_seqlens[b + 1] - start;
  float* cs = state + (size_t)slot_ids[b] * dm.state_stride + dm.conv_off;
  const int keep = dm.taps - 1;
  // entry m holds the input (keep - m) tokens before the next one; ascending m reads entries that
  // are not yet overwritten
  for (int m = 0; m < keep; ++m) {
    const int i = n - keep + m;
    cs[(size_t)m * dm.channels + ch] =
        i >= 0 ? to_f32(proj[(size_t)(start + i) * ld + ch]) : cs[(size_t)(m + n) * dm.channels + ch];
  }
}

constexpr int kLanesPerColumn = 4;
constexpr int kColumnsPerBlock = 32;

template <int DPER>
__global__ void __launch_bounds__(kLanesPerColumn * kColumnsPerBlock)
delta_recurrence_kernel(const float* __restrict__ qn, const float* __restrict__ kn,
                        const float* __restrict__ v, const float* __restrict__ g,
                        const float* __restrict__ beta, float* __restrict__ state,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                        DeltaDims dm, float* __restrict__ o) {
  const int b = blockIdx.x / dm.H, h = blockIdx.x - b * dm.H;
  const int part = threadIdx.x & (kLanesPerColumn - 1);
  const int col = blockIdx.y * kColumnsPerBlock + (threadIdx.x >> 2);
  pdl_trigger();
  pdl_wait();
  const int D = dm.D, Vd = dm.Vd;
  const int row0 = part * DPER;                    // this lane's rows: row0 .. row0 + DPER - 1
  const bool col_ok = col < Vd;
  const int cj = col_ok ? col : 0;
  const int kvh = h / (dm.H / dm.G);
  float* Sg = state + (size_t)slot_ids[b] * dm.state_stride + ((size_t)h * D) * Vd + cj;
  float S[DPER];
#pragma unroll
  for (int i = 0; i < DPER; ++i) S[i] = (row0 + i < D) ? Sg[(size_t)(row0 + i) * Vd] : 0.f;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const size_t GD = (size_t)dm.G * D, HD = (size_t)dm.H * D, HV = (size_t)dm.H * Vd;
  float kc[DPER], qc[DPER], gc[DPER], vc, bc;
  auto fetch = [&](int t, float (&k_)[DPER], float (&q_)[DPER], float (&g_)[DPER], float& v_,
                   float& b_) {
    const float* kp = kn + (size_t)t * GD + (size_t)kvh * D + row0;
    const float* qp = qn + (size_t)t * GD + (size_t)kvh * D + row0;
    const float* gp = g + (size_t)t * HD + (size_t)h * D + row0;
#pragma unroll
    for (int i = 0; i < DPER; ++i) {
      const bool ok = row0 + i < D;
      k_[i] = ok ? kp[i] : 0.f;
      q_[i] = ok ? qp[i] : 0.f;
      g_[i] = ok ? gp[i] : 0.f;
    }
    v_ = v[(size_t)t * HV + (size_t)h * Vd + cj];
    b_ = beta[(size_t)t * dm.H + h];
  };
  if (t0 < t1) fetch(t0, kc, qc, gc, vc, bc);
  for (int t = t0; t < t1; ++t) {
    float kx[DPER], qx[DPER], gx[DPER], vx = 0.f, bx = 0.f;
    if (t + 1 < t1) fetch(t + 1, kx, qx, gx, vx, bx);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < DPER; ++i) {
      S[i] *= gc[i];
      dot = fmaf(S[i], kc[i], dot);
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    const float u = bc * (vc - dot);
    float out = 0.f;
#pragma unroll
    for (int i = 0; i < DPER; ++i) {
      S[i] = fmaf(kc[i], u, S[i]);
      out = fmaf(S[i], qc[i], out);
    }
    out += __shfl_xor_sync(0xffffffffu, out, 1);
    out += __shfl_xor_sync(0xffffffffu, out, 2);
    if (part == 0 && col_ok) o[(size_t)t * HV + (size_t)h * Vd + col] = out;
    if (t + 1 < t1) {
#pragma unroll
      for (int i = 0; i < DPER; ++i) kc[i] = kx[i], qc[i] = qx[i], gc[i] = gx[i];
      vc = vx, bc = bx;
    }
  }
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < DPER; ++i)
      if (row0 + i < D) Sg[(size_t)(row0 + i) * Vd] = S[i];
  }
}

template <typename T>
__global__ void delta_output_kernel(const float* __restrict__ o, const T* __restrict__ gate,
                                    int gate_ld, const float* __restrict__ w, float eps,
                                    T* __restrict__ out, int pairs, int H, int Vd) {
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  if (pair >= pairs) return;
  const int t = pair / H, h = pair - t * H;
  const float* src = o + (size_t)pair * Vd;
  float ss = 0.f;
  for (int j = lane; j < Vd; j += 32) ss += src[j] * src[j];
  ss = warp_sum(ss);
  const float rms = sqrtf(ss / (float)Vd + eps);
  for (int j = lane; j < Vd; j += 32) {
    const float gt = sigmoid_f(to_f32(gate[(size_t)t * gate_ld + (size_t)h * Vd + j]));
    out[(size_t)pair * Vd + j] = from_f32<T>(src[j] / rms * w[j] * gt);
  }
}

}  // namespace gf

using namespace gf;
using bf = __nv_bfloat16;

GF_DEFINE_PDL_SWITCH

static DeltaDims dims_of(int H, int G, int D, int Vd, int taps, int state_stride, int conv_off) {
  DeltaDims dm;
  dm.H = H, dm.G = G, dm.D = D, dm.Vd = Vd, dm.taps = taps;
  dm.channels = 2 * G * D + H * Vd;
  dm.state_stride = state_stride, dm.conv_off = conv_off;
  return dm;
}

// proj: [T, ld] with the columns q | k | v first and the H beta columns at b_off.
GF_EXPORT int gf_delta_prepare(const void* proj, int ld, int b_off, const float* a,
                               const float* conv_w, const float* dt_bias, const float* A_log,
                               float* state, const int* seq_of_token, const int* cu_seqlens,
                               const int* slot_ids, int T, int B, int H, int G, int D, int Vd,
                               int taps, int state_stride, int conv_off, float* qn, float* kn,
                               float* v, float* g, float* beta, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (H % G || taps < 1) return -3;
  const DeltaDims dm = dims_of(H, G, D, Vd, taps, state_stride, conv_off);
  const size_t smem = (size_t)dm.channels * sizeof(float);
  if (smem > 160 * 1024) return -3;
  auto st = (cudaStream_t)stream;
  static OncePerDevice once;
  int rc = once.run([] {
    cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(delta_prepare_kernel<bf>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
  });
  if (rc) return rc;
  if (dtype == GF_F32)
    rc = launch_kernel(delta_prepare_kernel<float>, dim3(T), dim3(256), smem, st,
                       (const float*)proj, ld, b_off, a, conv_w, dt_bias, A_log,
                       (const float*)state, seq_of_token, cu_seqlens, slot_ids, dm, qn, kn, v, g,
                       beta);
  else
    rc = launch_kernel(delta_prepare_kernel<bf>, dim3(T), dim3(256), smem, st, (const bf*)proj, ld,
                       b_off, a, conv_w, dt_bias, A_log, (const float*)state, seq_of_token,
                       cu_seqlens, slot_ids, dm, qn, kn, v, g, beta);
  if (rc || taps == 1) return rc;
  const dim3 grid((dm.channels + 127) / 128, B);
  if (dtype == GF_F32)
    return launch_kernel(delta_conv_state_kernel<float>, grid, dim3(128), 0, st,
                         (const float*)proj, ld, state, cu_seqlens, slot_ids, dm);
  return launch_kernel(delta_conv_state_kernel<bf>, grid, dim3(128), 0, st, (const bf*)proj, ld,
                       state, cu_seqlens, slot_ids, dm);
}

GF_EXPORT int gf_delta_recurrence(const float* qn, const float* kn, const float* v, const float* g,
                                  const float* beta, float* state, const int* cu_seqlens,
                                  const int* slot_ids, int B, int H, int G, int D, int Vd,
                                  int state_stride, float* o, void* stream) {
  if (B <= 0) return 0;
  if (H % G) return -3;
  const DeltaDims dm = dims_of(H, G, D, Vd, 1, state_stride, 0);
  auto st = (cudaStream_t)stream;
  const dim3 grid(B * H, (Vd + kColumnsPerBlock - 1) / kColumnsPerBlock);
  const dim3 block(kLanesPerColumn * kColumnsPerBlock);
#define GF_GO(DPER)                                                                            \
  if (D <= kLanesPerColumn * DPER)                                                             \
    return launch_kernel(delta_recurrence_kernel<DPER>, grid, block, 0, st, qn, kn, v, g, beta, \
                         state, cu_seqlens, slot_ids, dm, o)
  GF_GO(4);
  GF_GO(8);
  GF_GO(16);
  GF_GO(32);
  GF_GO(64);
#undef GF_GO
  return -3;
}

GF_EXPORT int gf_delta_output(const float* o, const void* gate, int gate_ld, const float* w,
                              float eps, void* out, int T, int H, int Vd, int dtype, void* stream) {
  const int pairs = T * H;
  if (pairs <= 0) return 0;
  auto st = (cudaStream_t)stream;
  const dim3 grid((pairs + 3) / 4), block(128);
  if (dtype == GF_F32)
    return launch_kernel(delta_output_kernel<float>, grid, block, 0, st, o, (const float*)gate,
                         gate_ld, w, eps, (float*)out, pairs, H, Vd);
  return launch_kernel(delta_output_kernel<bf>, grid, block, 0, st, o, (const bf*)gate, gate_ld, w,
                       eps, (bf*)out, pairs, H, Vd);
}
