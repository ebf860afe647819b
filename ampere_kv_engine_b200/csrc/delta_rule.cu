// The gated delta rule: a mixer whose memory is one float32 matrix S [dim, vdim] per head and request.
//
//   delta_prep:  one product holds [q | k | v | gate | beta | step] of every token.  q, k and v pass a short causal
//                convolution over the sequence's own earlier tokens (the inputs before the step's first token come
//                from the request's state slot) and SiLU; q and k heads become unit vectors (q also times
//                dim^-1/2); beta = sigmoid(.), decay = exp(-exp(rate_log) * softplus(step + step_bias)).
//                Everything it writes is float32.  One warp per (token, head).
//   delta_scan:  one block per (sequence, head) walks the step's tokens of that sequence in order:
//                S *= decay;  u = beta (v - S^T k);  S += k u^T;  o = S^T q.
//                A thread group of L lanes owns one value column of S (dim / L elements per lane, in registers for
//                the whole step); the two products are EPT multiply-adds per lane and a shuffle reduction over the
//                group; the next token's q, k, v, beta, decay are fetched while the current one is computed, so a
//                token costs one block barrier.  Afterwards the block's warps apply the output norm
//                o / sqrt(mean(o^2) + eps) * w * silu(gate) to the tokens in parallel, and the block of head 0 moves
//                the sequence's last taps - 1 convolution inputs into the state.
//
// The walk is token by token whatever the step holds, so the state after a token does not depend on how the
// tokens were cut into steps.  A sequence whose state slot is negative (padding of a captured step) is left alone
// and its output rows are zero.
#include "common.cuh"
#include "launchers.h"

namespace akv {

namespace {

__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// the sequence s with cu_q[s] <= token < cu_q[s + 1]
__device__ __forceinline__ int sequence_of(const int32_t* cu_q, int num_seqs, int64_t token) {
  int lo = 0, hi = num_seqs;          // invariant: cu_q[lo] <= token < cu_q[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_q[mid] <= token) lo = mid; else hi = mid;
  }
  return lo;
}

constexpr int kMaxPerLane = kDeltaMaxDim / 32;

}  // namespace

template <typename T>
__global__ void delta_prep_kernel(DeltaParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int G = p.num_kv_heads, H = p.num_heads, D = p.head_dim, V = p.v_dim;
  const int units = 2 * G + H + 1;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= p.num_tokens * units) return;
  const int64_t token = item / units;
  const int unit = (int)(item - token * units);
  const int channels = 2 * G * D + H * V;
  const int64_t width = (int64_t)channels + (int64_t)H * V + 2 * H;
  const T* x = (const T*)p.x;
  const int s = sequence_of(p.cu_q, p.num_seqs, token);
  const int slot = p.state_slots[s];
  float* coef = p.coef + token * 2 * H;
  if (unit == units - 1) {
    for (int h = lane; h < H; h += 32) {
      float beta = 0.f, decay = 0.f;
      if (slot >= 0 && slot < p.num_slots) {
        const T* tail = x + token * width + channels + (int64_t)H * V;
        beta = 1.f / (1.f + expf(-to_float<T>(tail[h])));
        decay = expf(-expf(p.rate_log[h]) * softplus(to_float<T>(tail[H + h]) + p.step_bias[h]));
      }
      coef[h] = beta;
      coef[H + h] = decay;
    }
    return;
  }
  // a head of q, k or v: channels [first, first + n)
  const bool unit_vector = unit < 2 * G;
  const int n = unit_vector ? D : V;
  const int first = unit_vector ? unit * D : 2 * G * D + (unit - 2 * G) * V;
  float* out = p.qkv + token * channels + first;
  if (slot < 0 || slot >= p.num_slots) {
    for (int d = lane; d < n; d += 32) out[d] = 0.f;
    return;
  }
  const int64_t seq_first = p.cu_q[s];
  const int offset = (int)(token - seq_first);               // tokens of this sequence before this one in the step
  const int taps = p.taps;
  const float* before = p.state + (int64_t)slot * p.state_stride + p.memory;     // [taps - 1, channels]
  float vals[kMaxPerLane];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < kMaxPerLane; ++r) {
    const int d = lane + 32 * r;
    vals[r] = 0.f;
    if (d < n) {
      const int c = first + d;
      const float* w = p.conv + (int64_t)c * taps;
      float y = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int back = offset - (taps - 1) + j;            // index within the step's tokens of this sequence
        const float in = back >= 0 ? to_float<T>(x[(seq_first + back) * width + c])
                                   : before[(int64_t)(taps - 1 + back) * channels + c];
        y += w[j] * in;
      }
      y = y / (1.f + expf(-y));
      vals[r] = y;
      ss += y * y;
    }
  }
  float scale = 1.f;
  if (unit_vector) {
    scale = rsqrtf(warp_sum(ss) + p.unit_eps);
    if (unit < G) scale *= rsqrtf((float)D);
  }
#pragma unroll
  for (int r = 0; r < kMaxPerLane; ++r) {
    const int d = lane + 32 * r;
    if (d < n) out[d] = vals[r] * scale;
  }
}

int launch_delta_prep(const DeltaParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0) return 0;
  if (p.head_dim > kDeltaMaxDim || p.v_dim > kDeltaMaxDim || p.taps < 1 || p.taps > kDeltaMaxTaps)
    return (int)cudaErrorInvalidValue;
  const int units = 2 * p.num_kv_heads + p.num_heads + 1;
  const int warps = 4;
  const int64_t blocks = (p.num_tokens * units + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(delta_prep_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                             dim3(1, 1, 1), p);
  return (int)launch_chain(delta_prep_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, dim3(1, 1, 1), p);
}

// Shared memory of the scan, per buffer: q and k (each lane's EPT elements padded by four floats, so that the lanes
// of a group read different banks), v, beta and decay.
template <int EPT>
struct ScanLayout {
  static constexpr int kPitch = EPT + 4;
  __host__ __device__ static int vec(int lanes) { return lanes * kPitch; }
  // a multiple of four floats, so that the second buffer's rows can be read as float4 too
  __host__ __device__ static int floats(int lanes, int v_dim) { return (2 * vec(lanes) + v_dim + 2 + 3) / 4 * 4; }
};

template <typename T, int EPT>
__global__ void __launch_bounds__(EPT <= 32 ? 1024 : (EPT <= 64 ? 512 : 256)) delta_scan_kernel(DeltaParams p, int lanes) {
  extern __shared__ __align__(16) float smem[];
  using Layout = ScanLayout<EPT>;
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y;
  const int G = p.num_kv_heads, H = p.num_heads, D = p.head_dim, V = p.v_dim;
  const int channels = 2 * G * D + H * V;
  const int64_t width = (int64_t)channels + (int64_t)H * V + 2 * H;
  const int64_t first = p.cu_q[s];
  const int n = (int)(p.cu_q[s + 1] - first);
  const int slot = p.state_slots[s];
  const T* x = (const T*)p.x;
  T* out = (T*)p.out;
  if (n <= 0) return;
  if (slot < 0 || slot >= p.num_slots) {
    for (int64_t i = threadIdx.x; i < (int64_t)n * V; i += blockDim.x)
      out[(first + i / V) * H * V + (int64_t)h * V + i % V] = from_float<T>(0.f);
    return;
  }
  float* state = p.state + (int64_t)slot * p.state_stride;
  const int col = threadIdx.x / lanes, l = threadIdx.x % lanes;
  const bool owner = col < V;
  const int g = h / (H / G);
  // this lane's part of the column: elements [l * EPT, l * EPT + EPT) of the dim
  float S[EPT];
  float* mine = state + ((int64_t)h * V + col) * D + l * EPT;
#pragma unroll
  for (int e = 0; e < EPT; ++e) S[e] = (owner && l * EPT + e < D) ? mine[e] : 0.f;

  const int per_buffer = Layout::floats(lanes, V);
  // what a thread fetches for the next token: entries idx = threadIdx.x + k * blockDim.x of [q | k | v | beta | decay]
  const int fetch_total = 2 * D + V + 2;
  constexpr int kFetch = 8;           // at most 2 * 256 + 256 + 2 entries over at least 128 threads
  auto fetch = [&](int64_t token, float (&regs)[kFetch]) {
    const float* qkv = p.qkv + token * channels;
    const float* coef = p.coef + token * 2 * H;
#pragma unroll
    for (int k = 0; k < kFetch; ++k) {
      const int idx = threadIdx.x + k * blockDim.x;
      float v = 0.f;
      if (idx < D) v = qkv[g * D + idx];
      else if (idx < 2 * D) v = qkv[G * D + g * D + (idx - D)];
      else if (idx < 2 * D + V) v = qkv[2 * G * D + h * V + (idx - 2 * D)];
      else if (idx == 2 * D + V) v = coef[h];
      else if (idx == 2 * D + V + 1) v = coef[H + h];
      regs[k] = v;
    }
  };
  auto stash = [&](float* buffer, const float (&regs)[kFetch]) {
#pragma unroll
    for (int k = 0; k < kFetch; ++k) {
      const int idx = threadIdx.x + k * blockDim.x;
      if (idx < D) buffer[idx / EPT * Layout::kPitch + idx % EPT] = regs[k];
      else if (idx < 2 * D) buffer[Layout::vec(lanes) + (idx - D) / EPT * Layout::kPitch + (idx - D) % EPT] = regs[k];
      else if (idx < fetch_total) buffer[2 * Layout::vec(lanes) + (idx - 2 * D)] = regs[k];
    }
  };
  // rows of q and k beyond dim stay zero in both buffers
  for (int i = threadIdx.x; i < 2 * per_buffer; i += blockDim.x) smem[i] = 0.f;
  __syncthreads();
  float regs[kFetch];
  fetch(first, regs);
  stash(smem, regs);
  __syncthreads();
  float* scratch = p.scratch + first * H * V + (int64_t)h * V;
  for (int t = 0; t < n; ++t) {
    const float* buffer = smem + (t & 1) * per_buffer;
    if (t + 1 < n) fetch(first + t + 1, regs);
    const float* q = buffer + l * Layout::kPitch;
    const float* k = buffer + Layout::vec(lanes) + l * Layout::kPitch;
    const float* rest = buffer + 2 * Layout::vec(lanes);
    const float v = owner ? rest[col] : 0.f;
    const float beta = rest[V], decay = rest[V + 1];
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; e += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(k + e);
      S[e] *= decay; S[e + 1] *= decay; S[e + 2] *= decay; S[e + 3] *= decay;
      a0 += S[e] * kk.x; a1 += S[e + 1] * kk.y; a2 += S[e + 2] * kk.z; a3 += S[e + 3] * kk.w;
    }
    float kv = (a0 + a1) + (a2 + a3);
    for (int o = lanes >> 1; o > 0; o >>= 1) kv += __shfl_xor_sync(0xffffffffu, kv, o);
    const float u = beta * (v - kv);
    a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; e += 4) {
      const float4 kk = *reinterpret_cast<const float4*>(k + e);
      const float4 qq = *reinterpret_cast<const float4*>(q + e);
      S[e] += kk.x * u; S[e + 1] += kk.y * u; S[e + 2] += kk.z * u; S[e + 3] += kk.w * u;
      a0 += S[e] * qq.x; a1 += S[e + 1] * qq.y; a2 += S[e + 2] * qq.z; a3 += S[e + 3] * qq.w;
    }
    float o = (a0 + a1) + (a2 + a3);
    for (int w = lanes >> 1; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
    if (owner && l == 0) scratch[(int64_t)t * H * V + col] = o;
    if (t + 1 < n) stash(smem + ((t + 1) & 1) * per_buffer, regs);
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < EPT; ++e)
    if (owner && l * EPT + e < D) mine[e] = S[e];

  // the output norm and gate, a warp per token (the raw outputs of this block are visible to it after the barrier)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int64_t gate_first = (int64_t)channels + (int64_t)h * V;
  for (int t = warp; t < n; t += warps) {
    const float* raw = scratch + (int64_t)t * H * V;
    float ss = 0.f;
    for (int j = lane; j < V; j += 32) ss += raw[j] * raw[j];
    const float inv = rsqrtf(warp_sum(ss) / (float)V + p.norm_eps);
    const T* gate = x + (first + t) * width + gate_first;
    T* dst = out + (first + t) * H * V + (int64_t)h * V;
    for (int j = lane; j < V; j += 32) {
      const float z = to_float<T>(gate[j]);
      dst[j] = from_float<T>(raw[j] * inv * p.norm_weight[j] * (z / (1.f + expf(-z))));
    }
  }

  // the convolutions' memory: the last taps - 1 inputs of [what was there before | this step's rows]
  if (h == 0 && p.taps > 1) {
    const int keep = p.taps - 1;
    float* before = state + p.memory;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
      for (int i = 0; i < keep; ++i) {          // ascending: entry i reads entry i + n > i, not yet overwritten
        const int back = n - keep + i;          // index within the step's tokens of this sequence
        before[(int64_t)i * channels + c] = back >= 0 ? to_float<T>(x[(first + back) * width + c])
                                                       : before[(int64_t)(i + n) * channels + c];
      }
    }
  }
}

// (elements per lane, lanes per column) for a head of these sizes, or (0, 0) if no form of the kernel takes them
static void scan_shape(int dim, int v_dim, int& ept, int& lanes) {
  for (int e : {8, 16, 32, 64, 128}) {
    int l = 1;
    while (l * e < dim) l *= 2;
    const int limit = e <= 32 ? 1024 : (e <= 64 ? 512 : 256);
    if (l <= 32 && (v_dim * l + 31) / 32 * 32 <= limit) {
      ept = e;
      lanes = l;
      return;
    }
  }
  ept = lanes = 0;
}

bool delta_scan_supported(int dim, int v_dim) {
  int ept, lanes;
  scan_shape(dim, v_dim, ept, lanes);
  return ept != 0 && dim <= kDeltaMaxDim && v_dim <= kDeltaMaxDim;
}

template <typename T, int EPT>
static int launch_scan(const DeltaParams& p, int lanes, cudaStream_t stream) {
  // at least 128 threads: the fetch of a token's operands is spread over the block (threads without a column idle)
  const int threads = max(128, (p.v_dim * lanes + 31) / 32 * 32);
  const size_t smem = 2 * (size_t)ScanLayout<EPT>::floats(lanes, p.v_dim) * sizeof(float);
  auto kernel = delta_scan_kernel<T, EPT>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  return (int)launch_chain(kernel, dim3((unsigned)p.num_seqs, (unsigned)p.num_heads), dim3(threads), smem, stream,
                           dim3(1, 1, 1), p, lanes);
}

int launch_delta_scan(const DeltaParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0 || p.num_seqs == 0) return 0;
  int ept, lanes;
  scan_shape(p.head_dim, p.v_dim, ept, lanes);
  if (ept == 0 || p.head_dim > kDeltaMaxDim || p.v_dim > kDeltaMaxDim || p.num_heads > 65535)
    return (int)cudaErrorInvalidValue;
#define AKV_SCAN(E)                                                                           \
  case E:                                                                                     \
    return p.dtype == kBFloat16 ? launch_scan<__nv_bfloat16, E>(p, lanes, stream) : launch_scan<float, E>(p, lanes, stream)
  switch (ept) {
    AKV_SCAN(8);
    AKV_SCAN(16);
    AKV_SCAN(32);
    AKV_SCAN(64);
    AKV_SCAN(128);
  }
#undef AKV_SCAN
  return (int)cudaErrorInvalidValue;
}

}  // namespace akv
