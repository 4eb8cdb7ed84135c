// Latent attention: every token keeps ONE latent vector c (C channels, RMS-normed) and one rotated
// key part r (R channels) shared by all heads.  With the key up-projection folded into the query
// (q_lat = W_uk^T q_plain) a head's score against key j is (q_lat . c_j + q_rot . r_j) * scale and
// its output is sum_j p_j c_j (C channels), which the value up-projection turns into the head's
// values afterwards: multi-query attention with keys [c | r] and values c.
//
//   latent_prepare_kernel   per token: c = rmsnorm(first C of the down-projection) * w into the
//                           token's cache slot, the rotated key part into its slot, the heads'
//                           rotated query parts in fp32.  Rotation: channels (2i, 2i+1) of the first
//                           `rot` channels by the angle float(p) * freq[i], fp32.
//   latent_attention_kernel one block per (token, 8 heads), a warp a head; keys lo..p (lo = max(0,
//                           p - window + 1) with a window) visited in groups of 32 from lo, staged
//                           once per block in shared memory as fp32; running maximum, sum and the
//                           C-wide accumulator in fp32.  A row's result depends only on (lo, p) and
//                           the cache, never on how the step was cut or what else is in the batch.
#include "common.cuh"

namespace gf {

constexpr int kLatWarps = 8;        // heads per block
constexpr int kLatTile = 32;        // keys per tile (a lane a key)
constexpr int kLatMaxC = 512;       // latent channels a lane can accumulate (16 registers)

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ qd, int ld, int H, int D, int R, int C,
                                      int rot, const float* __restrict__ freq,
                                      const float* __restrict__ cnorm_w, float eps,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ slot_mapping, T* __restrict__ c_pages,
                                      T* __restrict__ r_pages, float* __restrict__ q_rot) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const T* row = qd + (size_t)t * ld;
  const T* dkv = row + (size_t)H * (D + R);
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  const float p = (float)positions[t];
  // the latent vector
  float ss = 0.f;
  for (int j = threadIdx.x; j < C; j += blockDim.x) {
    const float v = to_f32(dkv[j]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)C + eps);
  if (slot >= 0) {
    T* cdst = c_pages + (size_t)slot * C;
    for (int j = threadIdx.x; j < C; j += blockDim.x)
      cdst[j] = from_f32<T>(to_f32(dkv[j]) / rms * cnorm_w[j]);
  }
  // rotated parts: unit u < H is a head's query part, unit H the shared key part
  const int half = rot >> 1;
  for (int i = threadIdx.x; i < (H + 1) * half; i += blockDim.x) {
    const int u = i / half, k = i - u * half;
    const T* src = u < H ? row + (size_t)u * (D + R) + D : dkv + C;
    float sn, cs;
    sincosf(p * freq[k], &sn, &cs);
    const float a = to_f32(src[2 * k]), b = to_f32(src[2 * k + 1]);
    const float lo = a * cs - b * sn, hi = b * cs + a * sn;
    if (u < H) {
      float* dst = q_rot + ((size_t)t * H + u) * R;
      dst[2 * k] = lo;
      dst[2 * k + 1] = hi;
    } else if (slot >= 0) {
      T* dst = r_pages + (size_t)slot * R;
      dst[2 * k] = from_f32<T>(lo);
      dst[2 * k + 1] = from_f32<T>(hi);
    }
  }
  const int tail = R - rot;                       // channels that pass unrotated
  for (int i = threadIdx.x; i < (H + 1) * tail; i += blockDim.x) {
    const int u = i / tail, k = rot + (i - u * tail);
    if (u < H)
      q_rot[((size_t)t * H + u) * R + k] = to_f32(row[(size_t)u * (D + R) + D + k]);
    else if (slot >= 0)
      r_pages[(size_t)slot * R + k] = dkv[C + k];
  }
}

template <typename T>
__global__ void latent_attention_kernel(const float* __restrict__ q_lat,   // [H, T, C]
                                        const float* __restrict__ q_rot,   // [T, H, R]
                                        const T* __restrict__ c_pages, const T* __restrict__ r_pages,
                                        const int* __restrict__ block_table, int table_stride,
                                        const int* __restrict__ seq_of_token,
                                        const int* __restrict__ positions, T* __restrict__ out,
                                        int num_tokens, int H, int C, int R, int page_size,
                                        int window, float scale) {
  extern __shared__ float smem[];
  const int Dk = C + R, ks = Dk + 1;               // odd stride: a lane a key without conflicts
  float* keys = smem;                              // [kLatTile][ks]
  float* qs = smem + kLatTile * ks;                // [kLatWarps][Dk]
  __shared__ int slots[kLatTile];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * kLatWarps + warp;
  const bool live = h < H;
  pdl_trigger();
  pdl_wait();
  const int b = seq_of_token[t];
  const int p = positions[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* tbl = block_table + (size_t)b * table_stride;
  if (live) {
    const float* ql = q_lat + ((size_t)h * num_tokens + t) * C;
    const float* qr = q_rot + ((size_t)t * H + h) * R;
    float* q = qs + warp * Dk;
    for (int d = lane; d < C; d += 32) q[d] = ql[d];
    for (int d = lane; d < R; d += 32) q[C + d] = qr[d];
  }
  float acc[kLatMaxC / 32];
#pragma unroll
  for (int i = 0; i < kLatMaxC / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int c0 = lo; c0 <= p; c0 += kLatTile) {
    const int nvalid = min(kLatTile, p - c0 + 1);
    __syncthreads();                               // the tile before is no longer read
    if (threadIdx.x < kLatTile) {
      const int c = c0 + threadIdx.x;
      slots[threadIdx.x] = c <= p ? tbl[c / page_size] * page_size + c % page_size : 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nvalid * Dk; i += blockDim.x) {
      const int j = i / Dk, d = i - j * Dk;
      const size_t s = (size_t)slots[j];
      keys[j * ks + d] = d < C ? to_f32(c_pages[s * C + d]) : to_f32(r_pages[s * R + (d - C)]);
    }
    __syncthreads();
    if (live) {
      const float* q = qs + warp * Dk;
      const bool valid = lane < nvalid;
      float s = -INFINITY;
      if (valid) {
        const float* k = keys + lane * ks;
        float dot = 0.f;
        for (int d = 0; d < Dk; ++d) dot = fmaf(q[d], k[d], dot);
        s = dot * scale;
      }
      const float m_new = fmaxf(m, warp_max(s));
      const float pexp = valid ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);
      l = l * corr + warp_sum(pexp);
#pragma unroll
      for (int i = 0; i < kLatMaxC / 32; ++i) acc[i] *= corr;
      for (int j = 0; j < nvalid; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pexp, j);
        const float* v = keys + j * ks;
#pragma unroll
        for (int i = 0; i < kLatMaxC / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < C) acc[i] = fmaf(pj, v[d], acc[i]);
        }
      }
      m = m_new;
    }
  }
  if (live) {
    T* o = out + ((size_t)h * num_tokens + t) * C;
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < kLatMaxC / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < C) o[d] = from_f32<T>(acc[i] * inv);
    }
  }
}

}  // namespace gf

using namespace gf;
using bf = __nv_bfloat16;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_latent_prepare(const void* qd, int ld, int H, int D, int R, int C, int rot,
                                const float* freq, const float* cnorm_w, float eps,
                                const int* positions, const int* slot_mapping, void* c_pages,
                                void* r_pages, float* q_rot, int T, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (rot % 2 || rot > R) return -3;
  auto st = (cudaStream_t)stream;
  if (dtype == GF_F32)
    return launch_kernel(latent_prepare_kernel<float>, dim3(T), dim3(128), 0, st, (const float*)qd,
                         ld, H, D, R, C, rot, freq, cnorm_w, eps, positions, slot_mapping,
                         (float*)c_pages, (float*)r_pages, q_rot);
  return launch_kernel(latent_prepare_kernel<bf>, dim3(T), dim3(128), 0, st, (const bf*)qd, ld, H,
                       D, R, C, rot, freq, cnorm_w, eps, positions, slot_mapping, (bf*)c_pages,
                       (bf*)r_pages, q_rot);
}

GF_EXPORT int gf_latent_attention(const float* q_lat, const float* q_rot, const void* c_pages,
                                  const void* r_pages, const int* block_table, int table_stride,
                                  const int* seq_of_token, const int* positions, void* out, int T,
                                  int H, int C, int R, int page_size, int window, float scale,
                                  int dtype, void* stream) {
  if (T <= 0) return 0;
  if (C > kLatMaxC || C <= 0 || R < 0) return -3;
  const int Dk = C + R;
  const size_t smem = ((size_t)kLatTile * (Dk + 1) + (size_t)kLatWarps * Dk) * sizeof(float);
  if (smem > 200 * 1024) return -3;
  auto st = (cudaStream_t)stream;
  const dim3 grid(T, (H + kLatWarps - 1) / kLatWarps), block(kLatWarps * 32);
  static OncePerDevice once;
  const int rc = once.run([] {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<float>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(latent_attention_kernel<bf>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  });
  if (rc) return rc;
  if (dtype == GF_F32)
    return launch_kernel(latent_attention_kernel<float>, grid, block, smem, st, q_lat, q_rot,
                         (const float*)c_pages, (const float*)r_pages, block_table, table_stride,
                         seq_of_token, positions, (float*)out, T, H, C, R, page_size, window,
                         scale);
  return launch_kernel(latent_attention_kernel<bf>, grid, block, smem, st, q_lat, q_rot,
                       (const bf*)c_pages, (const bf*)r_pages, block_table, table_stride,
                       seq_of_token, positions, (bf*)out, T, H, C, R, page_size, window, scale);
}
