// Scored paged attention on the mma.sync tensor cores for rows that are key and value at once: a paged tensor of
// bfloat16 rows [pages, kv heads, page size, row stride], read whole (head_dim elements) as the key and in its first
// v_dim elements as the value, the layout of a cache that keeps one compressed latent per token.  Same mathematics and
// the same work items as the general kernel of scored_attention.cu (a CTA here where a warp stands there): 16 rows
// of a tile, rows being (token, head-in-group) pairs, one kv head, one key split.
//
// A CTA of four warps walks its key range 32 keys at a time.  The block's rows come into shared memory once
// (cp.async, two stages, 16-byte pieces, zero-filled past the range) and serve both products.  Scores: warp w takes a
// quarter of head_dim's 16-element steps against all 32 keys; its Q fragments stay in registers through the whole
// walk, and the four partial score tiles are added up through shared memory (one ldmatrix per two MMAs).
// Thread by thread the sums go through the score reshaping, the row maxima of the four warps meet in shared memory,
// P goes there as bfloat16, and for P V warp w owns the value dims v_dim / 4 * w ..: its accumulators (v_dim / 32
// tiles of 16 x 8) stay in registers.
// With several splits the partial (acc, max, sum) go to the workspace that scored_attention.cu's merge kernel reads.
#include "common.cuh"
#include "launchers.h"

#include <math_constants.h>

namespace akv {

namespace {

constexpr int kMmaKeys = 32;
constexpr int kMmaRows = 16;
constexpr int kPRow = 40;             // P row stride in elements: 80 bytes, an odd number of 16-byte pieces
constexpr int kMmaSteps = 9;          // most 16-element steps of the key width a warp takes: key widths up to 576
constexpr int kPartRow = 40;          // row stride of a partial score tile, in floats
constexpr float kLog2eF = 1.4426950408889634f;
constexpr float kLn2F = 0.6931471805599453f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory; `bytes` = 0 writes zeros and reads nothing
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Q [16][ldk] bfloat16 at first, then the four partial score tiles: the larger of the two, in 16-byte units
__host__ __device__ inline int first_region_bytes(int ldk) {
  const int q = kMmaRows * ldk * 2, parts = 4 * kMmaRows * kPartRow * 4;
  return ((q > parts ? q : parts) + 15) / 16 * 16;
}

}  // namespace

template <int DV>
__global__ void __launch_bounds__(128)
scored_attention_mma_kernel(ScoredAttentionParams sp, int row_groups, int ldk) {
  constexpr int NV = DV / 32;          // 8-dim value tiles per warp
  const PagedAttentionParams& p = sp.base;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int D = p.head_dim, NH = p.num_heads, NKV = p.num_kv_heads, G = NH / NKV, P = p.page_size;
  const int64_t item = blockIdx.x;
  const int rg = (int)(item % row_groups);
  const int kvh = (int)((item / row_groups) % NKV);
  const int split = (int)((item / ((int64_t)row_groups * NKV)) % p.num_splits);
  const int tile = (int)(item / ((int64_t)row_groups * NKV * p.num_splits));

  const int seq = p.tile_seq[tile];
  const int q0 = p.tile_q0[tile];
  const int nq = p.tile_nq[tile];
  const int rows_in_tile = nq * G;
  const int row0 = rg * kMmaRows;
  if (row0 >= rows_in_tile) return;
  const int nrows = min(kMmaRows, rows_in_tile - row0);
  const int ctx = p.ctx_lens[seq];
  const int seq_q0 = p.cu_q[seq];
  const int q_len = p.cu_q[seq + 1] - seq_q0;
  const int tile_pos = ctx - q_len + (q0 - seq_q0);

  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [16][ldk]; then the partial scores
  float* spart = reinterpret_cast<float*>(smem_raw);                              // [4][16][kPartRow]
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw + first_region_bytes(ldk));   // [2][32][ldk]
  __nv_bfloat16* ps = ks + 2 * kMmaKeys * ldk;                                    // [16][kPRow]
  float* smax = reinterpret_cast<float*>(ps + kMmaRows * kPRow);                  // [4][16]
  float* lsum = smax + 4 * kMmaRows;                                              // [4][16]

  const __nv_bfloat16* q = (const __nv_bfloat16*)p.q;
  for (int idx = tid; idx < kMmaRows * (D / 8); idx += 128) {
    const int r = idx / (D / 8), c = idx - r * (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows) {
      const int rr = row0 + r;
      v = *reinterpret_cast<const uint4*>(q + ((int64_t)(q0 + rr / G) * NH + kvh * G + rr % G) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(qs + r * ldk + c * 8) = v;
  }

  // this thread's two rows: g and g + 8
  const int g = lane >> 2;
  int pos[2], first_key[2];
  float slope[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    const bool live = row < nrows;
    pos[r] = live ? tile_pos + (row0 + row) / G : -1;
    int first = 0;
    if (live && p.window > 0) first = max(first, pos[r] - p.window + 1);
    if (live && sp.chunk > 0) first = max(first, pos[r] / sp.chunk * sp.chunk);
    first_key[r] = first;
    slope[r] = (live && sp.slopes != nullptr) ? sp.slopes[kvh * G + (row0 + row) % G] : 0.f;
  }
  const int pos_first = tile_pos + row0 / G;
  const int pos_last = tile_pos + (row0 + nrows - 1) / G;
  int lo_item = 0;
  if (p.window > 0) lo_item = max(lo_item, pos_first - p.window + 1);
  if (sp.chunk > 0) lo_item = max(lo_item, pos_first / sp.chunk * sp.chunk);
  const int hi_item = pos_last + 1;
  int per = (max(hi_item - lo_item, 0) + p.num_splits - 1) / p.num_splits;
  per = (per + kMmaKeys - 1) / kMmaKeys * kMmaKeys;
  const int start = lo_item + split * per;
  const int end = min(hi_item, start + per);
  const int num_blocks = end > start ? (end - start + kMmaKeys - 1) / kMmaKeys : 0;
  const float inv_cap = sp.softcap > 0.f ? 1.f / sp.softcap : 0.f;

  const __nv_bfloat16* rows = (const __nv_bfloat16*)p.k_cache;
  const int32_t* table = p.block_table + (int64_t)seq * p.table_width;
  const int pieces = D / 8;

  // Warp w fetches the block's keys 8 w .. 8 w + 7: lane i < 8 looks up the cache row of the i-th of them (one
  // division and one table read per block and lane), then all lanes copy each row's 16-byte pieces side by side.
  // (With the pieces dealt out thread by thread, each with its own division and look-up, the address arithmetic took
  // longer than the products.)
  auto load_block = [&](int b) {
    __nv_bfloat16* stage = ks + (b & 1) * kMmaKeys * ldk;
    const int key0 = start + b * kMmaKeys;
    int my_row = -1;
    if (lane < 8) {
      const int key = key0 + warp * 8 + lane;
      if (key < end) {
        const int logical = key / P;
        const int page = logical < p.table_width ? table[logical] : -1;
        if (page < 0 || page >= p.num_pages) set_status(p.status, kBadPage);
        else my_row = (page * NKV + kvh) * P + key % P;
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int row = __shfl_sync(0xffffffffu, my_row, i);
      const __nv_bfloat16* src = rows + (int64_t)(row < 0 ? 0 : row) * sp.k_row_stride;
      const uint32_t dst = smem_u32(stage + (warp * 8 + i) * ldk);
      const int bytes = row < 0 ? 0 : 16;
      for (int col = lane; col < pieces; col += 32) cp_async_16(dst + col * 16, src + col * 8, bytes);
    }
    cp_async_commit();
  };

  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};      // m in log2 units
  float o[NV][4];
#pragma unroll
  for (int v = 0; v < NV; ++v) o[v][0] = o[v][1] = o[v][2] = o[v][3] = 0.f;

  if (num_blocks > 0) load_block(0);
  // this warp's share of the key width: steps [step0, step0 + my_steps) of 16 elements, its Q fragments in registers
  const int steps = D / 16, per_warp = (steps + 3) / 4;
  const int step0 = warp * per_warp;
  const int my_steps = max(0, min(per_warp, steps - step0));
  uint32_t qa[kMmaSteps][4];
  __syncthreads();
  {
    const uint32_t q_addr = smem_u32(qs + (lane & 15) * ldk + (lane >> 4) * 8);
#pragma unroll
    for (int s = 0; s < kMmaSteps; ++s) {
      if (s < my_steps) ldsm_x4(q_addr + (step0 + s) * 32, qa[s]);
      else qa[s][0] = qa[s][1] = qa[s][2] = qa[s][3] = 0u;
    }
  }
  const int t2 = (lane & 3) * 2;
  const int mat = lane >> 3;
  for (int b = 0; b < num_blocks; ++b) {
    cp_async_wait_all();
    __syncthreads();                       // block b has landed; block b - 1 and Q in shared memory are used up
    if (b + 1 < num_blocks) load_block(b + 1);
    const __nv_bfloat16* stage = ks + (b & 1) * kMmaKeys * ldk;
    const int key0 = start + b * kMmaKeys;

    // this warp's part of the scores: all 32 keys against the 16 rows over its share of the key width
    float part[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) part[j][0] = part[j][1] = part[j][2] = part[j][3] = 0.f;
    // ldmatrix x4: matrices 0, 1 = keys 0-7 of a 16-key half at elements 0-7, 8-15 of the step; 2, 3 = keys 8-15
    const uint32_t k_addr = smem_u32(stage + ((mat >> 1) * 8 + (lane & 7)) * ldk + step0 * 16 + (mat & 1) * 8);
#pragma unroll
    for (int s = 0; s < kMmaSteps; ++s) {
      if (s < my_steps) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t kb[4];
          ldsm_x4(k_addr + (half * 16 * ldk + s * 16) * 2, kb);
          mma_16816(part[2 * half], qa[s], kb[0], kb[1]);
          mma_16816(part[2 * half + 1], qa[s], kb[2], kb[3]);
        }
      }
    }
    float* mine = spart + warp * kMmaRows * kPartRow;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      *reinterpret_cast<float2*>(mine + g * kPartRow + j * 8 + t2) = make_float2(part[j][0], part[j][1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * kPartRow + j * 8 + t2) = make_float2(part[j][2], part[j][3]);
    }
    __syncthreads();
    // the sums for this thread's two rows and two of warp w's eight keys
    float sc[4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float2 sum = make_float2(0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float2 v = *reinterpret_cast<const float2*>(spart + (w * kMmaRows + g + 8 * r) * kPartRow + warp * 8 + t2);
        sum.x += v.x;
        sum.y += v.y;
      }
      sc[2 * r] = sum.x;
      sc[2 * r + 1] = sum.y;
    }
    float bmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const int key = key0 + warp * 8 + (lane & 3) * 2 + (e & 1);
      const bool visible = key < end && key <= pos[r] && key >= first_key[r];
      float x = sc[e] * p.scale;
      if (sp.softcap > 0.f) x = sp.softcap * tanhf(x * inv_cap);
      x -= slope[r] * (float)(pos[r] - key);
      sc[e] = visible ? x * kLog2eF : -CUDART_INF_F;
      bmax[r] = fmaxf(bmax[r], sc[e]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 1));
      bmax[r] = fmaxf(bmax[r], __shfl_xor_sync(0xffffffffu, bmax[r], 2));
    }
    if ((lane & 3) == 0) {
      smax[warp * kMmaRows + g] = bmax[0];
      smax[warp * kMmaRows + g + 8] = bmax[1];
    }
    __syncthreads();
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = g + 8 * r;
      float mx = m[r];
#pragma unroll
      for (int w = 0; w < 4; ++w) mx = fmaxf(mx, smax[w * kMmaRows + row]);
      alpha[r] = (mx == -CUDART_INF_F) ? 1.f : exp2f(m[r] - mx);
      m[r] = mx;
      const float pa = sc[2 * r] == -CUDART_INF_F ? 0.f : exp2f(sc[2 * r] - mx);
      const float pb = sc[2 * r + 1] == -CUDART_INF_F ? 0.f : exp2f(sc[2 * r + 1] - mx);
      l[r] = l[r] * alpha[r] + pa + pb;
      *reinterpret_cast<__nv_bfloat162*>(ps + row * kPRow + warp * 8 + (lane & 3) * 2) = __floats2bfloat162_rn(pa, pb);
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      o[v][0] *= alpha[0];
      o[v][1] *= alpha[0];
      o[v][2] *= alpha[1];
      o[v][3] *= alpha[1];
    }
    __syncthreads();                       // P of all four warps is in place
    // O[:, this warp's value dims] += P V; a value is the first v_dim elements of the key row it shares
#pragma unroll
    for (int u = 0; u < kMmaKeys / 16; ++u) {
      uint32_t a[4];
      ldsm_x4(smem_u32(ps + (lane & 15) * kPRow + u * 16 + (lane >> 4) * 8), a);
      // ldmatrix x4 transposed: matrices 0, 1 = keys 0-7, 8-15 of the 16 at one 8-dim tile; 2, 3 = at the next tile
      const uint32_t v_addr = smem_u32(stage + (u * 16 + (mat & 1) * 8 + (lane & 7)) * ldk + warp * (DV / 4) + (mat >> 1) * 8);
#pragma unroll
      for (int v = 0; v < NV; v += 2) {
        uint32_t vb[4];
        ldsm_x4_trans(v_addr + v * 16, vb);
        mma_16816(o[v], a, vb[0], vb[1]);
        mma_16816(o[v + 1], a, vb[2], vb[3]);
      }
    }
  }

  // row sums: over the four lanes that share a row, then over the warps (each summed its own keys, in its own scale:
  // all warps hold the same m)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  __syncthreads();
  if ((lane & 3) == 0) {
    lsum[warp * kMmaRows + g] = l[0];
    lsum[warp * kMmaRows + g + 8] = l[1];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    if (row >= nrows) continue;
    const float total = (lsum[row] + lsum[kMmaRows + row]) + (lsum[2 * kMmaRows + row] + lsum[3 * kMmaRows + row]);
    const int rr = row0 + row;
    const int64_t out_row = (int64_t)(q0 + rr / G) * NH + kvh * G + rr % G;
    if (p.num_splits == 1) {
      float inv = total > 0.f ? 1.f / total : 0.f;
      if (sp.gate != nullptr) inv *= sp.gate[out_row];
      __nv_bfloat16* out = (__nv_bfloat16*)p.out + out_row * DV + warp * (DV / 4) + (lane & 3) * 2;
#pragma unroll
      for (int v = 0; v < NV; ++v)
        *reinterpret_cast<__nv_bfloat162*>(out + v * 8) = __floats2bfloat162_rn(o[v][2 * r] * inv, o[v][2 * r + 1] * inv);
    } else {
      float* part = p.partials + (out_row * p.num_splits + split) * (int64_t)(DV + 2);
      float* dst = part + warp * (DV / 4) + (lane & 3) * 2;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        dst[v * 8] = o[v][2 * r];
        dst[v * 8 + 1] = o[v][2 * r + 1];
      }
      if (warp == 0 && (lane & 3) == 0) {
        part[DV] = m[r] == -CUDART_INF_F ? -CUDART_INF_F : m[r] * kLn2F;
        part[DV + 1] = total;
      }
    }
  }
}

// bfloat16 rows that are key and value at once (k_cache == v_cache), key width a multiple of 16 up to 576, value
// width 64, 128, 256 or 512, rows that start on 16-byte boundaries.
bool scored_attention_mma_supported(const ScoredAttentionParams& sp) {
  const PagedAttentionParams& p = sp.base;
  if (p.dtype != kBFloat16 || p.k_cache != p.v_cache || sp.k_row_stride != sp.v_row_stride) return false;
  if (p.head_dim % 16 || p.head_dim < 16 || p.head_dim > 64 * kMmaSteps || sp.v_dim > p.head_dim) return false;
  if (sp.v_dim != 64 && sp.v_dim != 128 && sp.v_dim != 256 && sp.v_dim != 512) return false;
  if (sp.k_row_stride % 8 || reinterpret_cast<uintptr_t>(p.k_cache) % 16 || reinterpret_cast<uintptr_t>(p.q) % 16)
    return false;
  if (p.num_pages * p.num_kv_heads * (int64_t)p.page_size > 0x7fffffffLL) return false;     // row indices are 32-bit
  return true;
}

template <int DV>
static int launch_mma(const ScoredAttentionParams& sp, cudaStream_t stream) {
  const PagedAttentionParams& p = sp.base;
  const int G = p.num_heads / p.num_kv_heads;
  const int row_groups = (p.q_tile * G + kMmaRows - 1) / kMmaRows;
  const int64_t blocks = (int64_t)p.num_tiles * p.num_kv_heads * row_groups * p.num_splits;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const int ldk = p.head_dim + 8;
  const size_t smem = (size_t)first_region_bytes(ldk) + (size_t)2 * kMmaKeys * ldk * 2 + kMmaRows * kPRow * 2 +
                      8 * kMmaRows * sizeof(float);
  auto kernel = scored_attention_mma_kernel<DV>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
  }
  return (int)launch_chain(kernel, dim3((unsigned)blocks), dim3(128), smem, stream, dim3(1, 1, 1), sp, row_groups, ldk);
}

int launch_scored_attention_mma(const ScoredAttentionParams& sp, cudaStream_t stream) {
  switch (sp.v_dim) {
    case 64: return launch_mma<64>(sp, stream);
    case 128: return launch_mma<128>(sp, stream);
    case 256: return launch_mma<256>(sp, stream);
    case 512: return launch_mma<512>(sp, stream);
    default: return (int)cudaErrorInvalidValue;
  }
}

}  // namespace akv
