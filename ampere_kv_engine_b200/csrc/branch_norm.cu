// Row-wise kernels of layers whose branches are normed on the way out, and the gated activations beside SiLU.
//
//   add_layernorm:     hidden += delta (optional), then LayerNorm without a bias of every row, or of gathered rows:
//                      (x - mean) / sqrt(var + eps) * w with var = mean((x - mean)^2).
//   branch_layernorm:  hidden += LayerNorm(branch): the norm sits on the branch's output and its result is what
//                      joins the float32 residual stream; optionally the new stream rounded to the compute dtype.
//                      The branch may also come as the rows of routed experts that are still to be added up.
//   stream_copy:       the float32 stream rounded to the compute dtype (what the first branch of a model reads).
//   glu:               act(gate) * up with the tanh form of GELU, SiLU, or the clamped form
//                      g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(slope * g) * (u + 1).
//   softcap:           cap * tanh(x / cap) in place on float32 logits.
//
// One block per row; the row is held in shared memory between the passes (mean, squared deviations, output), so the
// variance is the two-pass one.  Means, variances, rsqrt, the weight and the sum are float; storage is T.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

// mean and 1 / sqrt(var + eps) of row_cache[0, n) (already filled by this block); every thread gets both
__device__ __forceinline__ void row_moments(const float* row_cache, int64_t n, float sum, float eps, float* scratch,
                                            float& mean, float& inv) {
  mean = block_sum(sum, scratch) / (float)n;
  float dev = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const float d = row_cache[i] - mean;
    dev += d * d;
  }
  inv = rsqrtf(block_sum(dev, scratch) / (float)n + eps);
}

int row_threads(int64_t hidden_size) {
  int threads = 32;
  while (threads < 512 && threads * 4 < hidden_size) threads *= 2;
  return threads;
}

}  // namespace

template <typename T, typename TD>
__global__ void add_layernorm_kernel(float* __restrict__ hidden, const TD* __restrict__ delta,
                                     const float* __restrict__ weight, T* __restrict__ out,
                                     const int32_t* __restrict__ rows, int64_t num_tokens, int64_t hidden_size,
                                     float eps, int* status) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t out_row = blockIdx.x;
  int64_t src = out_row;
  const bool gathered = rows != nullptr;
  if (gathered) {
    src = rows[out_row];
    if (src < 0 || src >= num_tokens) {
      if (threadIdx.x == 0) set_status(status, kBadRow);
      src = 0;
    }
  }
  float* h = hidden + src * hidden_size;
  const TD* d = delta ? delta + src * hidden_size : nullptr;
  float sum = 0.f;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    float v = h[i];
    if (d) {
      v += to_float<TD>(d[i]);
      if (!gathered) h[i] = v;
    }
    row_cache[i] = v;
    sum += v;
  }
  float mean, inv;
  row_moments(row_cache, hidden_size, sum, eps, scratch, mean, inv);
  T* o = out + out_row * hidden_size;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x)
    o[i] = from_float<T>((row_cache[i] - mean) * inv * weight[i]);
}

int launch_add_layernorm(float* hidden, const void* delta, const float* weight, void* out, const int32_t* rows,
                         int64_t num_rows, int64_t num_tokens, int64_t hidden_size, float eps, int dtype, int* status,
                         cudaStream_t stream) {
  const int64_t n = rows ? num_rows : num_tokens;
  if (n == 0) return 0;
  const size_t smem = (size_t)hidden_size * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const int threads = row_threads(hidden_size);
  auto launch = [&](auto kernel, auto* typed_delta, auto* typed_out) {
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
    }
    return (int)launch_chain(kernel, dim3((unsigned)n), dim3(threads), smem, stream, dim3(1, 1, 1), hidden, typed_delta,
                             weight, typed_out, rows, num_tokens, hidden_size, eps, status);
  };
  if (dtype == kBFloat16)
    return launch(add_layernorm_kernel<__nv_bfloat16, __nv_bfloat16>, (const __nv_bfloat16*)delta, (__nv_bfloat16*)out);
  return launch(add_layernorm_kernel<float, float>, (const float*)delta, (float*)out);
}

template <typename TB, typename TC>
__global__ void branch_layernorm_kernel(float* __restrict__ hidden, const TB* __restrict__ branch,
                                        const float* __restrict__ weight, TC* __restrict__ copy, int64_t hidden_size,
                                        float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const TB* b = branch + row * hidden_size;
  float sum = 0.f;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    const float v = to_float<TB>(b[i]);
    row_cache[i] = v;
    sum += v;
  }
  float mean, inv;
  row_moments(row_cache, hidden_size, sum, eps, scratch, mean, inv);
  float* h = hidden + row * hidden_size;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    const float v = h[i] + (row_cache[i] - mean) * inv * weight[i];
    h[i] = v;
    if (copy != nullptr) copy[row * hidden_size + i] = from_float<TC>(v);
  }
}

int launch_branch_layernorm(float* hidden, const void* branch, int branch_dtype, const float* weight, void* copy,
                            int copy_dtype, int64_t num_tokens, int64_t hidden_size, float eps, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const size_t smem = (size_t)hidden_size * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const int threads = row_threads(hidden_size);
  auto launch = [&](auto kernel, auto* typed_branch, auto* typed_copy) {
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
    }
    return (int)launch_chain(kernel, dim3((unsigned)num_tokens), dim3(threads), smem, stream, dim3(1, 1, 1), hidden,
                             typed_branch, weight, typed_copy, hidden_size, eps);
  };
  const bool bf_copy = copy != nullptr && copy_dtype == kBFloat16;
  if (copy != nullptr && !bf_copy) return (int)cudaErrorInvalidValue;   // a float32 copy is the stream itself
  if (branch_dtype == kBFloat16) {
    if (bf_copy)
      return launch(branch_layernorm_kernel<__nv_bfloat16, __nv_bfloat16>, (const __nv_bfloat16*)branch,
                    (__nv_bfloat16*)copy);
    return launch(branch_layernorm_kernel<__nv_bfloat16, float>, (const __nv_bfloat16*)branch, (float*)nullptr);
  }
  if (bf_copy)
    return launch(branch_layernorm_kernel<float, __nv_bfloat16>, (const float*)branch, (__nv_bfloat16*)copy);
  return launch(branch_layernorm_kernel<float, float>, (const float*)branch, (float*)nullptr);
}

// The same with the branch given as float32 rows that are still to be added up: row t of the branch is
// parts[t * top], ..., parts[t * top + top - 1] in that order, plus shared[t] (or nothing).
template <typename TS, typename TC>
__global__ void branch_layernorm_parts_kernel(float* __restrict__ hidden, const float* __restrict__ parts, int top,
                                              const TS* __restrict__ shared, const float* __restrict__ weight,
                                              TC* __restrict__ copy, int64_t hidden_size, float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const float* first = parts + row * top * hidden_size;
  float sum = 0.f;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < top; ++s) v += first[s * hidden_size + i];
    if (shared != nullptr) v += to_float<TS>(shared[row * hidden_size + i]);
    row_cache[i] = v;
    sum += v;
  }
  float mean, inv;
  row_moments(row_cache, hidden_size, sum, eps, scratch, mean, inv);
  float* h = hidden + row * hidden_size;
  for (int64_t i = threadIdx.x; i < hidden_size; i += blockDim.x) {
    const float v = h[i] + (row_cache[i] - mean) * inv * weight[i];
    h[i] = v;
    if (copy != nullptr) copy[row * hidden_size + i] = from_float<TC>(v);
  }
}

int launch_branch_layernorm_parts(float* hidden, const float* parts, int top, const void* shared, int shared_dtype,
                                  const float* weight, void* copy, int copy_dtype, int64_t num_tokens,
                                  int64_t hidden_size, float eps, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const size_t smem = (size_t)hidden_size * sizeof(float);
  if (smem > 200 * 1024 || top < 1) return (int)cudaErrorInvalidValue;
  const int threads = row_threads(hidden_size);
  auto launch = [&](auto kernel, auto* typed_shared, auto* typed_copy) {
    if (smem > 48 * 1024) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
    }
    return (int)launch_chain(kernel, dim3((unsigned)num_tokens), dim3(threads), smem, stream, dim3(1, 1, 1), hidden,
                             parts, top, typed_shared, weight, typed_copy, hidden_size, eps);
  };
  const bool bf_copy = copy != nullptr && copy_dtype == kBFloat16;
  if (copy != nullptr && !bf_copy) return (int)cudaErrorInvalidValue;
  if (shared != nullptr && shared_dtype == kBFloat16) {
    if (bf_copy)
      return launch(branch_layernorm_parts_kernel<__nv_bfloat16, __nv_bfloat16>, (const __nv_bfloat16*)shared,
                    (__nv_bfloat16*)copy);
    return launch(branch_layernorm_parts_kernel<__nv_bfloat16, float>, (const __nv_bfloat16*)shared, (float*)nullptr);
  }
  if (bf_copy)
    return launch(branch_layernorm_parts_kernel<float, __nv_bfloat16>, (const float*)shared, (__nv_bfloat16*)copy);
  return launch(branch_layernorm_parts_kernel<float, float>, (const float*)shared, (float*)nullptr);
}

__global__ void stream_copy_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (idx >= total) return;
  if (idx + 4 <= total && (reinterpret_cast<uintptr_t>(in) % 16 == 0) && (reinterpret_cast<uintptr_t>(out) % 8 == 0)) {
    const float4 v = *reinterpret_cast<const float4*>(in + idx);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(out + idx) = raw;
    return;
  }
  for (int64_t i = idx; i < min(idx + 4, total); ++i) out[i] = __float2bfloat16_rn(in[i]);
}

int launch_stream_copy(const float* in, void* out, int64_t total, cudaStream_t stream) {
  if (total == 0) return 0;
  const int threads = 256;
  const int64_t blocks = ((total + 3) / 4 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return (int)launch_chain(stream_copy_kernel, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1), in,
                           (__nv_bfloat16*)out, total);
}

__device__ __forceinline__ float glu_value(float g, float u, int kind, float limit, float slope) {
  if (kind == kGluSilu) return g / (1.f + expf(-g)) * u;
  if (kind == kGluGeluTanh) return activation_value(g, kActGeluTanh) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-slope * g)) * (u + 1.f);
}

template <typename T>
__global__ void glu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t inter, int64_t total,
                           int64_t block, int kind, float limit, float slope) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t token = idx / inter, i = idx - token * inter;
  const T* row = gate_up + token * 2 * inter;
  // gate and up columns alternate in runs of `block` (block == inter: all gate columns, then all up columns)
  const int64_t gi = i / block * 2 * block + i % block, ui = gi + block;
  out[idx] = from_float<T>(glu_value(to_float<T>(row[gi]), to_float<T>(row[ui]), kind, limit, slope));
}

int launch_glu(const void* gate_up, void* out, int64_t num_tokens, int64_t inter, int64_t block, int kind, float limit,
               float slope, int dtype, cudaStream_t stream) {
  const int64_t total = num_tokens * inter;
  if (total == 0) return 0;
  if (block <= 0 || inter % block != 0 || kind < kGluSilu || kind > kGluClampedSwish) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (dtype == kBFloat16)
    return (int)launch_chain(glu_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1),
                             (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total, block, kind, limit, slope);
  return (int)launch_chain(glu_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1),
                           (const float*)gate_up, (float*)out, inter, total, block, kind, limit, slope);
}

__global__ void softcap_kernel(float* __restrict__ x, int64_t total, float cap, float inv_cap) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx < total) x[idx] = cap * tanhf(x[idx] * inv_cap);
}

int launch_softcap(float* x, int64_t total, float cap, cudaStream_t stream) {
  if (total == 0) return 0;
  if (!(cap > 0.f)) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  return (int)launch_chain(softcap_kernel, dim3((unsigned)blocks), dim3(threads), 0, stream, dim3(1, 1, 1), x, total, cap,
                           1.f / cap);
}

}  // namespace akv
