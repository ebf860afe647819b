// Row-wise kernels between a mixer's projections and its attention, and a feed-forward's
// activation: what the fused q/k kernel of qk_rope_write.cu is for the rotate-half mixer, for
// mixers with other shapes.
//
//   head_prep:     one product holds [q heads | k heads | v heads | one gate column per q head] of a token.
//                  q and k heads are scaled to unit RMS (no weight), v is blended with the values an earlier
//                  layer computed for the same token, k and v go to their cache slots, the gates through a
//                  sigmoid.
//   latent_prep:   one product holds [query latent | key/value latent | shared rotated key part].  Both latents
//                  get an RMS norm with a plain weight; the rotated part gets rotary positions (pairs of
//                  neighbouring dims); latent and rotated part are written side by side into the token's cache row.
//   rotate_pairs:  rotary positions on a column range of every head of a [tokens, heads, width] tensor, written to
//                  a column range of another such tensor.
//   activation:    relu(x)^2, tanh-form GELU or SiLU, element by element.
//
// Sums of squares, rsqrt, angles, cos/sin, sigmoid and the blend are float; storage is T.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

template <typename T>
__device__ __forceinline__ T* cache_row(T* cache, int slot, int page_size, int64_t num_pages, int heads, int head,
                                        int64_t row_stride, int* status) {
  const int page = slot / page_size, off = slot - page * page_size;
  if (slot < 0 || page >= num_pages) {
    if (slot >= 0) set_status(status, kBadSlot);
    return nullptr;
  }
  return cache + (((int64_t)page * heads + head) * page_size + off) * row_stride;
}

}  // namespace

// One warp per (token, unit); units: NH q heads, NKV k heads, NKV v heads, then one unit for all gates.
template <typename T>
__global__ void head_prep_kernel(HeadPrepParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int NH = p.num_heads, NKV = p.no_kv ? 0 : p.num_kv_heads, D = p.head_dim, DV = p.v_dim;
  const int units = NH + 2 * NKV + (p.gate_out != nullptr ? 1 : 0);
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= p.num_tokens * units) return;
  const int64_t token = item / units;
  const int unit = (int)(item - token * units);
  const int64_t width = (int64_t)NH * D + (int64_t)NKV * D + (int64_t)NKV * DV + (p.gate_out != nullptr ? NH : 0);
  const T* x = (const T*)p.x + token * width;
  const int slot = p.slots != nullptr ? p.slots[token] : -1;
  if (unit < NH + NKV) {
    // a q or k head: x / sqrt(mean(x^2) + eps)
    const bool is_q = unit < NH;
    const T* src = x + (is_q ? (int64_t)unit * D : (int64_t)NH * D + (int64_t)(unit - NH) * D);
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float v = to_float<T>(src[d]);
      ss += v * v;
    }
    const float inv = p.unit_norm ? rsqrtf(warp_sum(ss) / (float)D + p.eps) : 1.f;
    T* dst;
    if (is_q) {
      dst = (T*)p.q_out + (token * NH + unit) * (int64_t)D;
    } else {
      dst = p.k_cache != nullptr ? cache_row((T*)p.k_cache, slot, p.page_size, p.num_pages, NKV, unit - NH,
                                             p.k_row_stride, p.status)
                                 : nullptr;
    }
    if (dst == nullptr) return;
    const float* w = is_q ? p.q_weight : p.k_weight;
    if (w != nullptr) {
      for (int d = lane; d < D; d += 32) dst[d] = from_float<T>(to_float<T>(src[d]) * inv * w[d]);
    } else {
      for (int d = lane; d < D; d += 32) dst[d] = from_float<T>(to_float<T>(src[d]) * inv);
    }
    return;
  }
  if (unit < NH + 2 * NKV) {
    const int h = unit - NH - NKV;
    const T* src = x + (int64_t)NH * D + (int64_t)NKV * D + (int64_t)h * DV;
    const int64_t dense = (token * NKV + h) * (int64_t)DV;
    T* dst = p.v_cache != nullptr ? cache_row((T*)p.v_cache, slot, p.page_size, p.num_pages, NKV, h,
                                              p.v_row_stride, p.status)
                                  : nullptr;
    const float lam = p.blend_weight != nullptr ? *p.blend_weight : 0.f;
    for (int d = lane; d < DV; d += 32) {
      float v = to_float<T>(src[d]);
      if (p.v_keep != nullptr) ((T*)p.v_keep)[dense + d] = from_float<T>(v);
      if (p.v_other != nullptr) v = (1.f - lam) * v + lam * to_float<T>(((const T*)p.v_other)[dense + d]);
      if (dst != nullptr) dst[d] = from_float<T>(v);
    }
    return;
  }
  const T* src = x + (int64_t)NH * D + (int64_t)NKV * D + (int64_t)NKV * DV;
  for (int h = lane; h < NH; h += 32) p.gate_out[token * NH + h] = 1.f / (1.f + expf(-to_float<T>(src[h])));
}

int launch_head_prep(const HeadPrepParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  const int units = p.num_heads + (p.no_kv ? 0 : 2 * p.num_kv_heads) + (p.gate_out != nullptr ? 1 : 0);
  const int warps = 4;
  const int64_t blocks = (p.num_tokens * units + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(head_prep_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(head_prep_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, dim3(1, 1, 1), p);
}

// One block per (token, segment): 0 = query latent, 1 = key/value latent, 2 = rotated key part.  (A warp per segment
// walked a latent of several hundred elements in a dozen dependent rounds: 14 us for 8 tokens.)
template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(LatentPrepParams p) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t token = blockIdx.x / 3;
  const int segment = (int)(blockIdx.x - token * 3);
  const int64_t width = (int64_t)p.q_rank + p.kv_rank + p.rot_dim;
  const T* x = (const T*)p.x + token * width;
  const int slot = p.slots != nullptr ? p.slots[token] : -1;
  T* row = p.cache != nullptr ? cache_row((T*)p.cache, slot, p.page_size, p.num_pages, 1, 0, p.row_stride, p.status)
                              : nullptr;
  if (segment < 2) {
    const int n = segment == 0 ? p.q_rank : p.kv_rank;
    const T* src = x + (segment == 0 ? 0 : p.q_rank);
    const float* w = segment == 0 ? p.q_weight : p.kv_weight;
    T* dst = segment == 0 ? (T*)p.q_latent + token * (int64_t)p.q_rank : row;
    if (n == 0 || dst == nullptr) return;                  // the same for every thread of the block
    float ss = 0.f;
    for (int d = threadIdx.x; d < n; d += blockDim.x) {
      const float v = to_float<T>(src[d]);
      ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)n + p.eps);
    for (int d = threadIdx.x; d < n; d += blockDim.x) dst[d] = from_float<T>(to_float<T>(src[d]) * inv * w[d]);
    return;
  }
  if (row == nullptr) return;
  const T* src = x + p.q_rank + p.kv_rank;
  T* dst = row + p.kv_rank;
  const float position = (float)p.positions[token];
  const int pairs = p.rot_dim / 2, turning = p.rotary_dims / 2;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    float u = to_float<T>(src[2 * i]), v = to_float<T>(src[2 * i + 1]);
    if (i < turning) {
      float sn, cs;
      sincosf(position * p.inv_freq[i], &sn, &cs);
      const float a = u * cs - v * sn, b = v * cs + u * sn;
      u = a;
      v = b;
    }
    dst[2 * i] = from_float<T>(u);
    dst[2 * i + 1] = from_float<T>(v);
  }
  if ((p.rot_dim & 1) && threadIdx.x == 0) dst[p.rot_dim - 1] = src[p.rot_dim - 1];
}

int launch_latent_prep(const LatentPrepParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.rotary_dims > p.rot_dim || (p.rotary_dims & 1)) return (int)cudaErrorInvalidValue;
  const int64_t blocks = p.num_tokens * 3;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(latent_prep_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(128), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(latent_prep_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, dim3(1, 1, 1), p);
}

// One thread per (token, head, pair of the column range).
template <typename T>
__global__ void rotate_pairs_kernel(const T* __restrict__ in, T* __restrict__ out, const int32_t* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int64_t total, int heads, int cols,
                                    int rotary_dims, int64_t in_width, int in_offset, int64_t out_width,
                                    int out_offset) {
  pdl_launch_dependents();
  pdl_wait();
  const int pairs = (cols + 1) / 2;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int i = (int)(idx % pairs);
  const int64_t row = idx / pairs;              // token * heads + head
  const int64_t token = row / heads;
  const T* src = in + row * in_width + in_offset;
  T* dst = out + row * out_width + out_offset;
  if (2 * i + 1 >= cols) {                        // an odd last column passes unchanged
    dst[2 * i] = src[2 * i];
    return;
  }
  float u = to_float<T>(src[2 * i]), v = to_float<T>(src[2 * i + 1]);
  if (2 * i + 1 < rotary_dims) {
    float sn, cs;
    sincosf((float)positions[token] * inv_freq[i], &sn, &cs);
    const float a = u * cs - v * sn, b = v * cs + u * sn;
    u = a;
    v = b;
  }
  dst[2 * i] = from_float<T>(u);
  dst[2 * i + 1] = from_float<T>(v);
}

int launch_rotate_pairs(const void* in, void* out, const int32_t* positions, const float* inv_freq,
                        int64_t num_tokens, int heads, int cols, int rotary_dims, int64_t in_width, int in_offset,
                        int64_t out_width, int out_offset, int dtype, cudaStream_t stream) {
  const int64_t total = num_tokens * heads * ((cols + 1) / 2);
  if (total == 0) return 0;
  if (rotary_dims > cols || (rotary_dims & 1) || in_offset + cols > in_width || out_offset + cols > out_width)
    return (int)cudaErrorInvalidValue;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (dtype == kBFloat16)
    return (int)launch_chain(rotate_pairs_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                             dim3(1, 1, 1), (const __nv_bfloat16*)in, (__nv_bfloat16*)out, positions, inv_freq, total,
                             heads, cols, rotary_dims, in_width, in_offset, out_width, out_offset);
  return (int)launch_chain(rotate_pairs_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1),
                           (const float*)in, (float*)out, positions, inv_freq, total, heads, cols, rotary_dims,
                           in_width, in_offset, out_width, out_offset);
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t total, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (idx >= total) return;
  if (idx + 8 <= total && (reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) % (8 * sizeof(T)) == 0) {
    float v[8];
    load8<T>(in + idx, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = activation_value(v[i], kind);
    if constexpr (sizeof(T) == 2) {
      uint4 raw;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      *reinterpret_cast<uint4*>(out + idx) = raw;
    } else {
      *reinterpret_cast<float4*>(out + idx) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(out + idx + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    return;
  }
  for (int64_t i = idx; i < min(idx + 8, total); ++i) out[i] = from_float<T>(activation_value(to_float<T>(in[i]), kind));
}

int launch_activation(const void* in, void* out, int64_t total, int kind, int dtype, cudaStream_t stream) {
  if (total == 0) return 0;
  if (kind < kActReluSquared || kind > kActSilu) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  const int64_t blocks = ((total + 7) / 8 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (dtype == kBFloat16)
    return (int)launch_chain(activation_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream,
                             dim3(1, 1, 1), (const __nv_bfloat16*)in, (__nv_bfloat16*)out, total, kind);
  return (int)launch_chain(activation_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1),
                           (const float*)in, (float*)out, total, kind);
}

}  // namespace akv
