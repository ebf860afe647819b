// The gated delta rule: a mixer whose memory is one float32 matrix S [dim, vdim] per head and request.
//
//   delta_prep:  one product holds [q | k | v | gate | beta | step] of every token.  q, k and v pass a short causal
//                convolution over the sequence's own earlier tokens (the inputs before the step's first token come
//                from the request's state slot) and SiLU; q and k heads become unit vectors (q also times
//                dim^-1/2); beta = sigmoid(.), decay = exp(-exp(rate_log) * softplus(step + step_bias)).
//                Everything it writes is float32.  One warp per (token, head).
//   delta_scan:  blocks per (sequence, head, slice of the value columns) walk the step's tokens of that sequence in
//                order:  S *= decay;  u = beta (v - S^T k);  S += k u^T;  o = S^T q.
//                A thread group of up to 8 lanes owns one value column of S (in registers for the whole step); the
//                two products are a few multiply-adds per lane and a shuffle reduction over the group; tokens are
//                staged through shared memory in chunks, so a token costs no block barrier.  A second kernel applies
//                the output norm o / sqrt(mean(o^2) + eps) * w * silu(gate) to all tokens in parallel and, in further
//                blocks, moves each sequence's last taps - 1 convolution inputs into the state.
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

// ---------------------------------------------------------------------------------------------------------
// The scan.  A block owns `cols` value columns of one head of one sequence; a group of `lanes` (up to 8) lanes owns
// a column, each lane EPT consecutive elements of the dim, in registers for the whole step.  Tokens are staged in
// chunks: while the block walks the tokens of one chunk out of shared memory (no barrier between tokens: all a
// token needs from other threads is two shuffle reductions inside its lane group), the next chunk's q, k, v, beta
// and decay are already under way from global memory.
//
// S in the state slot, per head: element (column, lane, e) at ((e / 4) * (v_dim * lanes) + column * lanes + lane) * 4
// + e % 4, so that a warp's float4 accesses are consecutive; a head takes v_dim * lanes * EPT floats.
namespace {

struct ScanShape {
  int ept, lanes, cols, threads, chunk;   // elements per lane, lanes per column, columns and threads per block, tokens per chunk
};

// a thread stages up to kScanRounds entries of each of up to kScanChunk tokens (registers it holds of the chunk
// under way)
constexpr int kScanRounds = 3, kScanChunk = 16;

// floats of one staged token in shared memory: q and k (each lane's elements padded by four floats), the block's v
// columns, beta and decay; a multiple of four, so that every token's q and k can be read as float4
__host__ __device__ inline int scan_token_floats(int lanes, int ept, int cols) {
  return (2 * lanes * (ept + 4) + cols + 2 + 3) / 4 * 4;
}

__host__ __device__ inline int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p *= 2;
  return p;
}

// the smallest EPT of 4, 8, 16, 32 with which 8 lanes cover the dim; 256 threads a block.  (Narrower slices of the
// value columns, so that a single sequence's blocks cover all SMs, were measured and not kept: a block's time per
// token is the chain of one token's latencies whatever its width, 0.31 us at 16 and at 32 columns.)
inline ScanShape scan_shape(int dim, int v_dim) {
  ScanShape s{0, 0, 0, 0, 0};
  for (int e : {4, 8, 16, 32}) {
    const int lanes = pow2_at_least((dim + e - 1) / e);
    if (lanes <= 8) {
      s.ept = e;
      s.lanes = lanes;
      break;
    }
  }
  if (s.ept == 0) return s;
  s.cols = 256 / s.lanes;
  if (s.cols > v_dim) s.cols = v_dim;
  s.threads = (s.cols * s.lanes + 31) / 32 * 32;
  if (s.threads < 128) s.threads = 128;      // the fetch of a chunk is spread over the block (threads without a column idle)
  // a token's entries must fit in kScanRounds rounds of the block
  while (s.threads * kScanRounds < 2 * dim + s.cols + 2) s.threads += 32;
  // the chunk of a prompt: 16 tokens, 8 where a lane holds 32 elements (two buffers within 48 KB)
  const int per_token = scan_token_floats(s.lanes, s.ept, s.cols);
  s.chunk = kScanChunk;
  while (s.chunk > 1 && 2 * s.chunk * per_token * 4 > 48 * 1024) s.chunk /= 2;
  if (s.ept >= 32 && s.chunk > 8) s.chunk = 8;
  return s;
}

}  // namespace

bool delta_scan_supported(int dim, int v_dim) {
  return dim > 0 && v_dim > 0 && dim <= kDeltaMaxDim && v_dim <= kDeltaMaxDim && scan_shape(dim, v_dim).ept != 0;
}

int64_t delta_memory_floats(int num_heads, int dim, int v_dim) {
  const ScanShape s = scan_shape(dim, v_dim);
  return (int64_t)num_heads * v_dim * s.lanes * s.ept;
}

template <int EPT, int LANES, int CHUNK>
__global__ void __launch_bounds__(256) delta_scan_kernel(DeltaParams p, int cols) {
  constexpr int chunk = CHUNK;
  extern __shared__ __align__(16) float smem[];
  constexpr int kPitch = EPT + 4;      // a lane's elements of q or k, padded: the lanes of a group read different banks
  constexpr int lanes = LANES;
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols;
  const int G = p.num_kv_heads, H = p.num_heads, D = p.head_dim, V = p.v_dim;
  const int channels = 2 * G * D + H * V;
  const int64_t first = p.cu_q[s];
  const int n = (int)(p.cu_q[s + 1] - first);
  const int slot = p.state_slots[s];
  if (n <= 0) return;
  const int mine_cols = min(cols, V - col0);
  float* scratch = p.scratch + first * H * V + (int64_t)h * V + col0;
  if (slot < 0 || slot >= p.num_slots) {
    for (int i = threadIdx.x; i < n * mine_cols; i += blockDim.x) scratch[(int64_t)(i / mine_cols) * H * V + i % mine_cols] = 0.f;
    return;
  }
  float* state = p.state + (int64_t)slot * p.state_stride;
  const int col = threadIdx.x / lanes, l = threadIdx.x % lanes;
  const bool owner = col < mine_cols;
  const int g = h / (H / G);
  float S[EPT];
  float* mine = state + (int64_t)h * V * lanes * EPT + ((int64_t)(col0 + col) * lanes + l) * 4;
  const int64_t quad_stride = (int64_t)V * lanes * 4;
#pragma unroll
  for (int e = 0; e < EPT; e += 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (owner) v = *reinterpret_cast<const float4*>(mine + (e / 4) * quad_stride);
    S[e] = v.x; S[e + 1] = v.y; S[e + 2] = v.z; S[e + 3] = v.w;
  }

  constexpr int vec = lanes * kPitch;                                 // floats of one token's q (or k) in shared memory
  const int per_token = scan_token_floats(lanes, EPT, cols);      // q, k, v of the block's columns, beta, decay
  const int per_buffer = chunk * per_token;
  // What a thread stages of every token: entry i = threadIdx.x + round * blockDim.x of [q | k | v | beta | decay].
  // Where it comes from (a column of the token's qkv or coef row) and where it goes in the token's shared-memory row
  // are worked out once; a chunk is then one load per (round, token).
  const int fetch_per_token = 2 * D + mine_cols + 2;
  const float* src[kScanRounds];
  int src_stride[kScanRounds], dst[kScanRounds];
#pragma unroll
  for (int r = 0; r < kScanRounds; ++r) {
    const int i = threadIdx.x + r * blockDim.x;
    src[r] = nullptr;
    src_stride[r] = 0;
    dst[r] = 0;
    if (i < fetch_per_token) {
      const float* qkv = p.qkv + first * channels;
      const float* coef = p.coef + first * 2 * H;
      src_stride[r] = i < 2 * D + mine_cols ? channels : 2 * H;
      if (i < D) {
        src[r] = qkv + g * D + i;
        dst[r] = i / EPT * kPitch + i % EPT;
      } else if (i < 2 * D) {
        src[r] = qkv + G * D + g * D + (i - D);
        dst[r] = vec + (i - D) / EPT * kPitch + (i - D) % EPT;
      } else if (i < 2 * D + mine_cols) {
        src[r] = qkv + 2 * G * D + h * V + col0 + (i - 2 * D);
        dst[r] = 2 * vec + (i - 2 * D);
      } else {
        src[r] = coef + (i == 2 * D + mine_cols ? h : H + h);
        dst[r] = 2 * vec + cols + (i - 2 * D - mine_cols);
      }
    }
  }
  float regs[kScanRounds][CHUNK];
  auto fetch = [&](int t0, int count) {
#pragma unroll
    for (int r = 0; r < kScanRounds; ++r) {
#pragma unroll
      for (int t = 0; t < CHUNK; ++t) {
        regs[r][t] = 0.f;
        if (src[r] != nullptr && t < count) regs[r][t] = src[r][(int64_t)(t0 + t) * src_stride[r]];
      }
    }
  };
  auto stash = [&](float* buffer, int count) {
#pragma unroll
    for (int r = 0; r < kScanRounds; ++r) {
#pragma unroll
      for (int t = 0; t < CHUNK; ++t)
        if (src[r] != nullptr && t < count) buffer[t * per_token + dst[r]] = regs[r][t];
    }
  };
  // elements of q and k beyond the dim stay zero in both buffers
  for (int i = threadIdx.x; i < 2 * per_buffer; i += blockDim.x) smem[i] = 0.f;
  __syncthreads();
  fetch(0, min(chunk, n));
  stash(smem, min(chunk, n));
  __syncthreads();
  for (int t0 = 0; t0 < n; t0 += chunk) {
    const int count = min(chunk, n - t0), next = min(chunk, n - t0 - chunk);
    const float* buffer = smem + ((t0 / chunk) & 1) * per_buffer;
    if (next > 0) fetch(t0 + chunk, next);
    const float* row = buffer;
    float* o_row = scratch + (int64_t)t0 * H * V + col;
    // two tokens per round of the loop: the read-out of one token (o = S^T q and its reduction) has no successor in
    // the chain S -> S^T k -> u -> S and can be issued among the next token's instructions
#pragma unroll 2
    for (int t = 0; t < count; ++t, row += per_token, o_row += H * V) {
      const float* q = row + l * kPitch;
      const float* k = row + vec + l * kPitch;
      const float v = owner ? row[2 * vec + col] : 0.f;
      const float beta = row[2 * vec + cols], decay = row[2 * vec + cols + 1];
      float kr[EPT];
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int e = 0; e < EPT; e += 4) {
        const float4 kk = *reinterpret_cast<const float4*>(k + e);
        kr[e] = kk.x; kr[e + 1] = kk.y; kr[e + 2] = kk.z; kr[e + 3] = kk.w;
        a0 = fmaf(S[e], kk.x, a0); a1 = fmaf(S[e + 1], kk.y, a1); a2 = fmaf(S[e + 2], kk.z, a2); a3 = fmaf(S[e + 3], kk.w, a3);
      }
      float kv = ((a0 + a1) + (a2 + a3)) * decay;           // (decay S)^T k
#pragma unroll
      for (int o = lanes >> 1; o > 0; o >>= 1) kv += __shfl_xor_sync(0xffffffffu, kv, o);
      const float u = beta * (v - kv);
      a0 = a1 = a2 = a3 = 0.f;
#pragma unroll
      for (int e = 0; e < EPT; e += 4) {
        const float4 qq = *reinterpret_cast<const float4*>(q + e);
        S[e] = fmaf(kr[e], u, S[e] * decay); S[e + 1] = fmaf(kr[e + 1], u, S[e + 1] * decay);
        S[e + 2] = fmaf(kr[e + 2], u, S[e + 2] * decay); S[e + 3] = fmaf(kr[e + 3], u, S[e + 3] * decay);
        a0 = fmaf(S[e], qq.x, a0); a1 = fmaf(S[e + 1], qq.y, a1); a2 = fmaf(S[e + 2], qq.z, a2); a3 = fmaf(S[e + 3], qq.w, a3);
      }
      float o = (a0 + a1) + (a2 + a3);
#pragma unroll
      for (int w = lanes >> 1; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if (owner && l == 0) *o_row = o;
    }
    if (next > 0) stash(smem + (((t0 / chunk) + 1) & 1) * per_buffer, next);
    __syncthreads();
  }
  if (owner) {
#pragma unroll
    for (int e = 0; e < EPT; e += 4)
      *reinterpret_cast<float4*>(mine + (e / 4) * quad_stride) = make_float4(S[e], S[e + 1], S[e + 2], S[e + 3]);
  }
}

// What follows the scan, in one launch.  Blocks [0, norm_blocks): the output norm and gate, a warp per (token, head):
// o / sqrt(mean(o^2) + eps) * w * silu(gate).  The blocks after them: the convolutions' memory, a thread per
// (sequence, channel): the last taps - 1 inputs of [what was there before | this step's rows]; a thread reads all it
// needs before it writes.
template <typename T>
__global__ void __launch_bounds__(128) delta_finish_kernel(DeltaParams p, int norm_blocks, int channel_blocks) {
  pdl_launch_dependents();
  pdl_wait();
  const int H = p.num_heads, V = p.v_dim;
  const int channels = 2 * p.num_kv_heads * p.head_dim + H * V;
  const int64_t width = (int64_t)channels + (int64_t)H * V + 2 * H;
  const T* x = (const T*)p.x;
  if ((int)blockIdx.x < norm_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= p.num_tokens * H) return;
    const int64_t token = item / H;
    const int h = (int)(item - token * H);
    const float* raw = p.scratch + token * H * V + (int64_t)h * V;
    float ss = 0.f;
    for (int j = lane; j < V; j += 32) ss += raw[j] * raw[j];
    const float inv = rsqrtf(warp_sum(ss) / (float)V + p.norm_eps);
    const T* gate = x + token * width + channels + (int64_t)h * V;
    T* dst = (T*)p.out + token * H * V + (int64_t)h * V;
    for (int j = lane; j < V; j += 32) {
      const float z = to_float<T>(gate[j]);
      dst[j] = from_float<T>(raw[j] * inv * p.norm_weight[j] * (z / (1.f + expf(-z))));
    }
    return;
  }
  const int block = (int)blockIdx.x - norm_blocks;
  const int s = block / channel_blocks;
  const int c = (block - s * channel_blocks) * blockDim.x + threadIdx.x;
  const int64_t first = p.cu_q[s];
  const int n = (int)(p.cu_q[s + 1] - first);
  const int slot = p.state_slots[s];
  if (c >= channels || n <= 0 || slot < 0 || slot >= p.num_slots) return;
  const int keep = p.taps - 1;
  float* before = p.state + (int64_t)slot * p.state_stride + p.memory;
  float kept[kDeltaMaxTaps - 1];
#pragma unroll
  for (int i = 0; i < kDeltaMaxTaps - 1; ++i) {
    kept[i] = 0.f;
    if (i < keep) {
      const int back = n - keep + i;          // index within the step's tokens of this sequence
      kept[i] = back >= 0 ? to_float<T>(x[(first + back) * width + c]) : before[(int64_t)(i + n) * channels + c];
    }
  }
#pragma unroll
  for (int i = 0; i < kDeltaMaxTaps - 1; ++i)
    if (i < keep) before[(int64_t)i * channels + c] = kept[i];
}

template <int EPT, int LANES, int CHUNK>
static int launch_scan_chunk(const DeltaParams& p, const ScanShape& shape, cudaStream_t stream) {
  const int threads = shape.threads;
  const int per_token = scan_token_floats(shape.lanes, EPT, shape.cols);
  const size_t smem = 2 * (size_t)CHUNK * per_token * sizeof(float);
  auto kernel = delta_scan_kernel<EPT, LANES, CHUNK>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  const int splits = (p.v_dim + shape.cols - 1) / shape.cols;
  return (int)launch_chain(kernel, dim3((unsigned)p.num_seqs, (unsigned)p.num_heads, (unsigned)splits), dim3(threads),
                           smem, stream, dim3(1, 1, 1), p, shape.cols);
}

// Steps of about a token per sequence (decoding) stage two tokens at a time: fewer registers and less shared memory
// per block, so more blocks share an SM while the state streams through; prompts stage the largest chunk that fits.
template <int EPT, int LANES>
static int launch_scan(const DeltaParams& p, const ScanShape& shape, cudaStream_t stream) {
  constexpr int kLong = EPT >= 32 ? 8 : 16;
  if (p.num_tokens <= 2 * (int64_t)p.num_seqs) return launch_scan_chunk<EPT, LANES, 2>(p, shape, stream);
  if (shape.chunk < kLong) return (int)cudaErrorInvalidValue;
  return launch_scan_chunk<EPT, LANES, kLong>(p, shape, stream);
}

int launch_delta_scan(const DeltaParams& p, cudaStream_t stream) {
  if (p.num_tokens == 0 || p.num_seqs == 0) return 0;
  const ScanShape shape = scan_shape(p.head_dim, p.v_dim);
  if (shape.ept == 0 || p.head_dim > kDeltaMaxDim || p.v_dim > kDeltaMaxDim || p.num_heads > 65535 ||
      p.memory != delta_memory_floats(p.num_heads, p.head_dim, p.v_dim) || shape.threads > 256 ||
      shape.threads * kScanRounds < 2 * p.head_dim + shape.cols + 2 ||
      reinterpret_cast<uintptr_t>(p.state) % 16 != 0 || p.state_stride % 4 != 0)      // S moves as float4
    return (int)cudaErrorInvalidValue;
  int err;
  // more than four elements per lane only where eight lanes do not cover the dim otherwise
  if (shape.ept == 4) {
    switch (shape.lanes) {
      case 1: err = launch_scan<4, 1>(p, shape, stream); break;
      case 2: err = launch_scan<4, 2>(p, shape, stream); break;
      case 4: err = launch_scan<4, 4>(p, shape, stream); break;
      default: err = launch_scan<4, 8>(p, shape, stream); break;
    }
  } else if (shape.lanes != 8) {
    return (int)cudaErrorInvalidValue;
  } else if (shape.ept == 8) {
    err = launch_scan<8, 8>(p, shape, stream);
  } else if (shape.ept == 16) {
    err = launch_scan<16, 8>(p, shape, stream);
  } else {
    err = launch_scan<32, 8>(p, shape, stream);
  }
  if (err != 0) return err;
  const int warps = 4;
  const int64_t norm_blocks = (p.num_tokens * p.num_heads + warps - 1) / warps;
  const int channels = 2 * p.num_kv_heads * p.head_dim + p.num_heads * p.v_dim;
  const int channel_blocks = p.taps > 1 ? (channels + warps * 32 - 1) / (warps * 32) : 0;
  const int64_t blocks = norm_blocks + (int64_t)p.num_seqs * channel_blocks;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  if (p.dtype == kBFloat16)
    return (int)launch_chain(delta_finish_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                             dim3(1, 1, 1), p, (int)norm_blocks, channel_blocks);
  return (int)launch_chain(delta_finish_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, dim3(1, 1, 1),
                           p, (int)norm_blocks, channel_blocks);
}

}  // namespace akv
