// Gated delta rule with one decay per head and key channel, over packed tokens of several requests.
// A request's state lives in a slot: S [heads, D, Vd] in fp32 and the last (taps - 1) inputs of the
// short convolutions, fp32 as well.
//
//   delta_prepare_kernel     a warp a (token, head): causal convolution over time (taps from the rows of
//                            this step, or from the slot where the step's portion starts later than
//                            the tap reaches) + SiLU on the q | k | v channels; q and k made unit
//                            vectors per head (q also times D^-1/2); decay g = exp(-exp(A_log_h) *
//                            softplus(a + dt_bias)); beta = sigmoid(b).  Everything leaves in fp32.
//   delta_conv_state_kernel  a thread a (request, channel): the slot's last inputs after the step.
//   delta_recurrence_kernel  per (request, head): S <- g * S (rows); u = beta (v - S^T k);
//                            S <- S + k u^T; o = S^T q, token after token.  The columns of S are
//                            independent: four lanes or a warp share a column (a share of the rows
//                            each, in registers).  The tokens' operands come through two stages of
//                            shared memory, a chunk ahead (cp.async).
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

// A warp a (token, unit): units 0 .. G-1 are q heads, G .. 2G-1 k heads, then H v heads, then H
// decay rows, then one unit for the betas.  No warp waits for another.
template <typename T>
__device__ __forceinline__ float conv_silu_at(const T* __restrict__ proj, int ld, int r, int i,
                                              const float* __restrict__ cs,
                                              const float* __restrict__ conv_w, int taps, int CH,
                                              int ch) {
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int off = i - (taps - 1 - j);           // place of the tap's input in the portion
    const float x = off >= 0 ? to_f32(proj[(size_t)(r - (taps - 1 - j)) * ld + ch])
                             : cs[(size_t)(taps - 1 + off) * CH + ch];
    acc = fmaf(conv_w[(size_t)ch * taps + j], x, acc);
  }
  return acc * sigmoid_f(acc);
}

constexpr int kPrepareWarps = 8;
constexpr int kPrepareMaxPerLane = 8;              // head sizes up to 256

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
  const int r = blockIdx.x;
  const int unit = blockIdx.y * kPrepareWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  const int G = dm.G, H = dm.H, D = dm.D, Vd = dm.Vd;
  if (unit >= 2 * G + 2 * H + 1) return;
  const int b = seq_of_token[r];
  const int i = r - cu_seqlens[b];                // place in this step's portion
  const float* cs = state + (size_t)slot_ids[b] * dm.state_stride + dm.conv_off;
  const int taps = dm.taps, CH = dm.channels, GD = G * D;
  if (unit < 2 * G) {                             // a q or k head: convolve, activate, unit vector
    const int ch0 = unit * D;                     // q heads and k heads follow one another
    float y[kPrepareMaxPerLane];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kPrepareMaxPerLane; ++u) {
      const int d = lane + 32 * u;
      y[u] = d < D ? conv_silu_at(proj, ld, r, i, cs, conv_w, taps, CH, ch0 + d) : 0.f;
      ss += y[u] * y[u];
    }
    ss = warp_sum(ss);
    const bool is_q = unit < G;
    const float f = (is_q ? rsqrtf((float)D) : 1.f) / sqrtf(ss + 1e-6f);
    float* dst = (is_q ? qn : kn) + (size_t)r * GD + (size_t)(is_q ? unit : unit - G) * D;
#pragma unroll
    for (int u = 0; u < kPrepareMaxPerLane; ++u) {
      const int d = lane + 32 * u;
      if (d < D) dst[d] = y[u] * f;
    }
  } else if (unit < 2 * G + H) {                  // a v head
    const int h = unit - 2 * G;
    for (int j = lane; j < Vd; j += 32)
      v[((size_t)r * H + h) * Vd + j] =
          conv_silu_at(proj, ld, r, i, cs, conv_w, taps, CH, 2 * GD + h * Vd + j);
  } else if (unit < 2 * G + 2 * H) {              // a head's decays
    const int h = unit - 2 * G - H;
    const float rate = expf(A_log[h]);
    for (int d = lane; d < D; d += 32) {
      const size_t at = ((size_t)r * H + h) * D + d;
      g[at] = expf(-rate * softplus_f(a[at] + dt_bias[h * D + d]));
    }
  } else {
    for (int h = lane; h < H; h += 32)
      beta[(size_t)r * H + h] = sigmoid_f(to_f32(proj[(size_t)r * ld + b_off + h]));
  }
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

constexpr int kRecurrenceThreads = 128;
constexpr int kMaxColumnsPerBlock = 32;
constexpr int kStages = 3;             // chunks of tokens in shared memory

__device__ __forceinline__ void copy_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A block = (request, head, 128 / LP columns of S); LP lanes share a column, DPER rows each.  The
// tokens' k, q, g rows (padded to Dp = LP * DPER floats, the padding zero), the block's v columns and
// beta come through three stages of shared memory, CHUNK tokens each, asked for two chunks ahead
// with cp.async.  LP = 4 where requests x heads x columns fill the device (decode batches); LP = 32
// (a warp a column, eight columns a block) where they do not (one long prompt): a token is a chain
// of dependent instructions for a warp, and with eight times the lanes a column the chain is short
// and eight times as many warps share an SM's schedulers.
template <int DPER, int LP, int CHUNK, int THREADS>
__global__ void __launch_bounds__(THREADS)
delta_recurrence_kernel(const float* __restrict__ qn, const float* __restrict__ kn,
                        const float* __restrict__ v, const float* __restrict__ g,
                        const float* __restrict__ beta, float* __restrict__ state,
                        const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                        DeltaDims dm, float* __restrict__ o) {
  constexpr int Dp = LP * DPER;
  constexpr int kTok = 3 * Dp + kMaxColumnsPerBlock + 4;      // floats a token in a stage
  extern __shared__ __align__(16) float stage[];               // [kStages][CHUNK][kTok]
  constexpr int cols = THREADS / LP;
  const int b = blockIdx.x / dm.H, h = blockIdx.x - b * dm.H;
  const int part = threadIdx.x % LP, lc = threadIdx.x / LP;
  const int col0 = blockIdx.y * cols, col = col0 + lc;
  pdl_trigger();
  const int D = dm.D, Vd = dm.Vd;
  for (int i = threadIdx.x; i < kStages * CHUNK * kTok; i += blockDim.x) stage[i] = 0.f;
  __syncthreads();
  pdl_wait();
  const int row0 = part * DPER;
  const bool col_ok = col < Vd;
  const int cj = col_ok ? col : 0;
  const int kvh = h / (dm.H / dm.G);
  float* Sg = state + (size_t)slot_ids[b] * dm.state_stride + ((size_t)h * D) * Vd + cj;
  float S[DPER];
#pragma unroll
  for (int i = 0; i < DPER; ++i) S[i] = (row0 + i < D) ? Sg[(size_t)(row0 + i) * Vd] : 0.f;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  const size_t GD = (size_t)dm.G * D, HD = (size_t)dm.H * D, HV = (size_t)dm.H * Vd;
  const int ncols = min(cols, Vd - col0);
  // 16-byte copies where rows allow it (a thread keeps the same piece of every token), else 4-byte
  const bool vec = (D & 3) == 0 && (Vd & 3) == 0 && (ncols & 3) == 0;
  const int dq = D >> 2, pieces = 3 * dq + (ncols >> 2);
  auto ask = [&](int chunk) {                      // the chunk's tokens into stage chunk % kStages
    float* st = stage + (size_t)(chunk % kStages) * CHUNK * kTok;
    const int ta = t0 + chunk * CHUNK, n = min(CHUNK, t1 - ta);
    if (vec) {
      for (int e = threadIdx.x; e < pieces; e += blockDim.x) {
        const float* src;
        int dst, step;                             // source floats from one token to the next
        if (e < dq) src = kn + (size_t)ta * GD + (size_t)kvh * D + 4 * e, dst = 4 * e, step = (int)GD;
        else if (e < 2 * dq)
          src = qn + (size_t)ta * GD + (size_t)kvh * D + 4 * (e - dq), dst = Dp + 4 * (e - dq), step = (int)GD;
        else if (e < 3 * dq)
          src = g + (size_t)ta * HD + (size_t)h * D + 4 * (e - 2 * dq), dst = 2 * Dp + 4 * (e - 2 * dq),
          step = (int)HD;
        else
          src = v + (size_t)ta * HV + (size_t)h * Vd + col0 + 4 * (e - 3 * dq),
          dst = 3 * Dp + 4 * (e - 3 * dq), step = (int)HV;
        for (int tt = 0; tt < n; ++tt)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                           smem_u32(st + (size_t)tt * kTok + dst)),
                       "l"(src + (size_t)tt * step)
                       : "memory");
      }
      if (threadIdx.x < n)
        copy_async_4(st + (size_t)threadIdx.x * kTok + 3 * Dp + kMaxColumnsPerBlock,
                     beta + (size_t)(ta + threadIdx.x) * dm.H + h);
    } else {
      const int per = 3 * D + ncols + 1;
      for (int i = threadIdx.x; i < n * per; i += blockDim.x) {
        const int tt = i / per, e = i - tt * per;
        const size_t t = (size_t)(ta + tt);
        float* dst = st + (size_t)tt * kTok;
        if (e < D) copy_async_4(dst + e, kn + t * GD + (size_t)kvh * D + e);
        else if (e < 2 * D) copy_async_4(dst + Dp + (e - D), qn + t * GD + (size_t)kvh * D + (e - D));
        else if (e < 3 * D) copy_async_4(dst + 2 * Dp + (e - 2 * D), g + t * HD + (size_t)h * D + (e - 2 * D));
        else if (e < 3 * D + ncols)
          copy_async_4(dst + 3 * Dp + (e - 3 * D), v + t * HV + (size_t)h * Vd + col0 + (e - 3 * D));
        else copy_async_4(dst + 3 * Dp + kMaxColumnsPerBlock, beta + t * dm.H + h);
      }
    }
    copy_async_commit();
  };
  const int nchunks = (t1 - t0 + CHUNK - 1) / CHUNK;
  // two chunks are under way while a third is worked on (a group is committed every turn, empty
  // ones too, so that "all but the last two" always means "chunk c has landed")
  for (int c = 0; c < kStages - 1; ++c) {
    if (c < nchunks) ask(c);
    else copy_async_commit();
  }
  for (int c = 0; c < nchunks; ++c) {
    // the stage of chunk c + 2 held chunk c - 1, which every warp left at the last barrier
    if (c + kStages - 1 < nchunks) ask(c + kStages - 1);
    else copy_async_commit();
    copy_async_wait<kStages - 1>();
    __syncthreads();
    const float* st = stage + (size_t)(c % kStages) * CHUNK * kTok;
    const int ta = t0 + c * CHUNK, n = min(CHUNK, t1 - ta);
    // The chunk's tokens, unrolled: the read-out o = S^T q of a token is off the chain that the
    // next token waits for (only u is on it), so its lane reduction is left until the chunk is
    // done and the eight reductions run side by side.
    float outp[CHUNK];
#pragma unroll
    for (int tt = 0; tt < CHUNK; ++tt) {
      outp[tt] = 0.f;
      if (tt < n) {
        const float* tok = st + (size_t)tt * kTok;
        const float4* k4 = reinterpret_cast<const float4*>(tok + row0);
        const float4* q4 = reinterpret_cast<const float4*>(tok + Dp + row0);
        const float4* g4 = reinterpret_cast<const float4*>(tok + 2 * Dp + row0);
        const float vc = tok[3 * Dp + lc], bc = tok[3 * Dp + kMaxColumnsPerBlock];
        float kc[DPER];
#pragma unroll
        for (int i = 0; i < DPER / 4; ++i) {
          const float4 kk = k4[i], gg = g4[i];
          kc[4 * i] = kk.x, kc[4 * i + 1] = kk.y, kc[4 * i + 2] = kk.z, kc[4 * i + 3] = kk.w;
          S[4 * i] *= gg.x, S[4 * i + 1] *= gg.y, S[4 * i + 2] *= gg.z, S[4 * i + 3] *= gg.w;
        }
        float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < DPER; ++i) d4[i & 3] = fmaf(S[i], kc[i], d4[i & 3]);
        float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
#pragma unroll
        for (int sh = 1; sh < LP; sh <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sh);
        const float u = bc * (vc - dot);
        float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < DPER / 4; ++i) {
          const float4 qq = q4[i];
          S[4 * i] = fmaf(kc[4 * i], u, S[4 * i]);
          S[4 * i + 1] = fmaf(kc[4 * i + 1], u, S[4 * i + 1]);
          S[4 * i + 2] = fmaf(kc[4 * i + 2], u, S[4 * i + 2]);
          S[4 * i + 3] = fmaf(kc[4 * i + 3], u, S[4 * i + 3]);
          o4[0] = fmaf(S[4 * i], qq.x, o4[0]);
          o4[1] = fmaf(S[4 * i + 1], qq.y, o4[1]);
          o4[2] = fmaf(S[4 * i + 2], qq.z, o4[2]);
          o4[3] = fmaf(S[4 * i + 3], qq.w, o4[3]);
        }
        outp[tt] = (o4[0] + o4[1]) + (o4[2] + o4[3]);
      }
    }
#pragma unroll
    for (int sh = 1; sh < LP; sh <<= 1) {
#pragma unroll
      for (int tt = 0; tt < CHUNK; ++tt) outp[tt] += __shfl_xor_sync(0xffffffffu, outp[tt], sh);
    }
    if (part == 0 && col_ok) {
#pragma unroll
      for (int tt = 0; tt < CHUNK; ++tt)
        if (tt < n) o[(size_t)(ta + tt) * HV + (size_t)h * Vd + col] = outp[tt];
    }
    __syncthreads();                               // the stage is free for the chunk after next
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
  if (D > 32 * kPrepareMaxPerLane) return -3;
  auto st = (cudaStream_t)stream;
  const int units = 2 * G + 2 * H + 1;
  const dim3 pgrid(T, (units + kPrepareWarps - 1) / kPrepareWarps), pblock(kPrepareWarps * 32);
  int rc;
  if (dtype == GF_F32)
    rc = launch_kernel(delta_prepare_kernel<float>, pgrid, pblock, 0, st, (const float*)proj, ld,
                       b_off, a, conv_w, dt_bias, A_log, (const float*)state, seq_of_token,
                       cu_seqlens, slot_ids, dm, qn, kn, v, g, beta);
  else
    rc = launch_kernel(delta_prepare_kernel<bf>, pgrid, pblock, 0, st, (const bf*)proj, ld, b_off,
                       a, conv_w, dt_bias, A_log, (const float*)state, seq_of_token, cu_seqlens,
                       slot_ids, dm, qn, kn, v, g, beta);
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
  // few (request, head, column) triples: a warp (sixteen lanes for key sizes up to 64) a column
  // instead of four lanes (see the kernel)
  const bool wide = (long long)B * H * ((Vd + 31) / 32) < 2 * 148;
  const int lp = !wide ? 4 : (D <= 64 ? 16 : 32);
  const int threads = lp == 32 ? 256 : kRecurrenceThreads;
  const int cols = threads / lp;
  const dim3 grid(B * H, (Vd + cols - 1) / cols);
  const dim3 block(threads);
#define GF_GO(DPER, LP, CHUNK, THREADS)                                                            \
  if (lp == LP && D <= LP * DPER) {                                                                \
    const size_t smem =                                                                            \
        (size_t)kStages * CHUNK * (3 * LP * DPER + kMaxColumnsPerBlock + 4) * sizeof(float);       \
    return launch_kernel(delta_recurrence_kernel<DPER, LP, CHUNK, THREADS>, grid, block, smem, st,  \
                         qn, kn, v, g, beta, state, cu_seqlens, slot_ids, dm, o);                  \
  }
  GF_GO(4, 4, 8, kRecurrenceThreads)
  GF_GO(8, 4, 8, kRecurrenceThreads)
  GF_GO(16, 4, 8, kRecurrenceThreads)
  GF_GO(32, 4, 8, kRecurrenceThreads)
  GF_GO(64, 4, 4, kRecurrenceThreads)
  GF_GO(4, 16, 8, kRecurrenceThreads)
  GF_GO(4, 32, 8, 256)
  GF_GO(8, 32, 4, 256)
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
