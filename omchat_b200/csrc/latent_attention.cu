// Latent (compressed key/value) attention over a paged cache.
//
// What is cached per token and layer is ONE row shared by all heads: the normed latent c [r] followed by the rotated key part
// k_rot [dr]. The per-head key / value up-projections are absorbed into the query and the output:
//     score_h(i, j) = (q_h^nope W_uk,h) . c_j + q_h^rot . k_rot_j          o_h(i) = W_uv,h (sum_j p_h(i, j) c_j)
// so the attention kernel is multi-query attention with key width r + dr and value = the first r columns of the same row, and a
// key tile staged once serves as keys and as values. Kernels here:
//   omc_latent_kv_store  one CTA per new row: RMS norm of the latent, pairwise-interleaved rotation of the key part, append to the
//                        row's page (fused norm + rotation + cache write)
//   omc_rotary_q         the rotated query parts, written behind the absorbed part of each head
//   omc_latent_attn      plain kernel, any sizes, fp32 arithmetic: one CTA per (row, head), one warp per key, online softmax with
//                        an optional sink term exp(sink_h) that only enlarges the denominator
// Rows of a step are addressed by (slot, position): a row sees cache entries 0..position of its slot, whether they were written
// by this step or by earlier ones, so portions of prompts and single decoded tokens are the same case.
#include "seq_common.cuh"

namespace omc {

template <typename TW, typename TC>
__global__ void __launch_bounds__(128) latent_kv_store_kernel(const float* __restrict__ dkv, long long ld, int r, int dr,
                                                              const TW* __restrict__ w, float eps, const float* __restrict__ cs,
                                                              int rot_dims, const int32_t* __restrict__ pos,
                                                              const int32_t* __restrict__ slot,
                                                              const int32_t* __restrict__ block_table, int max_pages,
                                                              int page_size, TC* __restrict__ pool) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* row = dkv + (long long)t * ld;
  const int p = pos[t];
  const int page = block_table[(long long)slot[t] * max_pages + p / page_size];
  TC* dst = pool + ((long long)page * page_size + p % page_size) * (r + dr);
  float ss = 0.f;
  for (int c = threadIdx.x; c < r; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)r + eps);
  for (int c = threadIdx.x; c < r; c += blockDim.x) stf(dst + c, row[c] * rstd * ldf(w + c));
  const int half = rot_dims >> 1;
  const float* csr = cs + (long long)p * rot_dims;  // [half][2]
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = row[r + 2 * i], v = row[r + 2 * i + 1], co = csr[2 * i], si = csr[2 * i + 1];
    stf(dst + r + 2 * i, u * co - v * si);
    stf(dst + r + 2 * i + 1, v * co + u * si);
  }
  for (int c = rot_dims + threadIdx.x; c < dr; c += blockDim.x) stf(dst + r + c, row[r + c]);
}

template <typename TI, typename TQ>
__global__ void __launch_bounds__(128) rotary_q_kernel(const TI* __restrict__ q32, long long ldq, int H, int dn, int dr,
                                                       const float* __restrict__ cs, int rot_dims,
                                                       const int32_t* __restrict__ pos, TQ* __restrict__ qcat, int r) {
  const int t = blockIdx.x;
  const float* csr = cs + (long long)pos[t] * rot_dims;
  const int half = rot_dims >> 1;
  for (int h = 0; h < H; ++h) {
    const TI* src = q32 + (long long)t * ldq + (long long)h * (dn + dr) + dn;
    TQ* dst = qcat + ((long long)t * H + h) * (r + dr) + r;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float u = ldf(src + 2 * i), v = ldf(src + 2 * i + 1), co = csr[2 * i], si = csr[2 * i + 1];
      stf(dst + 2 * i, u * co - v * si);
      stf(dst + 2 * i + 1, v * co + u * si);
    }
    for (int c = rot_dims + threadIdx.x; c < dr; c += blockDim.x) stf(dst + c, ldf(src + c));
  }
}

// Both of the above for one row in one launch (a step's decode rows pay per launch, not per byte): the cache append of the row's
// latent and rotated key part, then the rotated query parts of all heads. All stored operands share one type.
template <typename T>
__global__ void __launch_bounds__(128) latent_rope_store_kernel(const float* __restrict__ dkv, long long ld, int r, int dr,
                                                                const T* __restrict__ w, float eps, const float* __restrict__ cs,
                                                                int rot_dims, const int32_t* __restrict__ pos,
                                                                const int32_t* __restrict__ slot,
                                                                const int32_t* __restrict__ block_table, int max_pages, int page_size,
                                                                T* __restrict__ pool, const T* __restrict__ q, long long ldq, int H, int dn,
                                                                T* __restrict__ qcat) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* row = dkv + (long long)t * ld;
  const int p = pos[t];
  const int page = block_table[(long long)slot[t] * max_pages + p / page_size];
  T* dst = pool + ((long long)page * page_size + p % page_size) * (r + dr);
  float ss = 0.f;
  for (int c = threadIdx.x; c < r; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)r + eps);
  for (int c = threadIdx.x; c < r; c += blockDim.x) stf(dst + c, row[c] * rstd * ldf(w + c));
  const int half = rot_dims >> 1;
  const float* csr = cs + (long long)p * rot_dims;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = row[r + 2 * i], v = row[r + 2 * i + 1], co = csr[2 * i], si = csr[2 * i + 1];
    stf(dst + r + 2 * i, u * co - v * si);
    stf(dst + r + 2 * i + 1, v * co + u * si);
  }
  for (int c = rot_dims + threadIdx.x; c < dr; c += blockDim.x) stf(dst + r + c, row[r + c]);
  // queries: every (head, pair) is one unit of work
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const T* src = q + (long long)t * ldq + (long long)h * (dn + dr) + dn;
    T* qd = qcat + ((long long)t * H + h) * (r + dr) + r;
    const float u = ldf(src + 2 * j), v = ldf(src + 2 * j + 1), co = csr[2 * j], si = csr[2 * j + 1];
    stf(qd + 2 * j, u * co - v * si);
    stf(qd + 2 * j + 1, v * co + u * si);
  }
  const int rest = dr - rot_dims;
  for (int i = threadIdx.x; i < H * rest; i += blockDim.x) {
    const int h = i / rest, c = rot_dims + (i - h * rest);
    stf(qcat + ((long long)t * H + h) * (r + dr) + r + c, ldf(q + (long long)t * ldq + (long long)h * (dn + dr) + dn + c));
  }
}

constexpr int kLatWarps = 4;
constexpr int kLatMaxPerLane = 32;  // r <= 1024

// One CTA per (row, head). Warp w takes keys w, w + 4, ...: lanes split the r + dr columns of the key row for the dot product,
// every lane keeps its share (columns lane, lane + 32, ...) of the running weighted sum of latents. The warps' partial
// (max, sum, accumulator) triples are merged through shared memory at the end.
template <typename TQ, typename TC>
__global__ void __launch_bounds__(kLatWarps * 32) latent_attn_kernel(const TQ* __restrict__ qcat, int H, int r, int dr,
                                                                     const TC* __restrict__ pool,
                                                                     const int32_t* __restrict__ block_table, int max_pages,
                                                                     int page_size, const int32_t* __restrict__ pos,
                                                                     const int32_t* __restrict__ slot,
                                                                     const float* __restrict__ sink, float scale,
                                                                     float* __restrict__ out) {
  extern __shared__ float sm[];  // q [r + dr] | acc [kLatWarps][r] | m [kLatWarps] | l [kLatWarps]
  const int t = blockIdx.x, h = blockIdx.y;
  const int D = r + dr;
  float* sq = sm;
  float* sacc = sm + D;
  float* s_m = sacc + kLatWarps * r;
  float* s_l = s_m + kLatWarps;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TQ* q = qcat + ((long long)t * H + h) * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) sq[c] = ldf(q + c);
  __syncthreads();
  const int n_keys = pos[t] + 1;
  const int32_t* bt = block_table + (long long)slot[t] * max_pages;
  float m = -INFINITY, l = 0.f;
  float acc[kLatMaxPerLane];
#pragma unroll
  for (int i = 0; i < kLatMaxPerLane; ++i) acc[i] = 0.f;
  for (int j = warp; j < n_keys; j += kLatWarps) {
    const TC* kr = pool + ((long long)bt[j / page_size] * page_size + j % page_size) * D;
    float d = 0.f;
    for (int c = lane; c < D; c += 32) d = fmaf(sq[c], ldf(kr + c), d);
    d = seq_warp_sum(d) * scale;
    const float mn = fmaxf(m, d);
    const float corr = expf(m - mn), pj = expf(d - mn);  // m = -inf on the first key: corr = 0
    l = l * corr + pj;
#pragma unroll
    for (int i = 0; i < kLatMaxPerLane; ++i) {
      const int c = lane + 32 * i;
      if (c < r) acc[i] = acc[i] * corr + pj * ldf(kr + c);
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < kLatMaxPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < r) sacc[warp * r + c] = acc[i];
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  __syncthreads();
  float mt = -INFINITY;
#pragma unroll
  for (int w = 0; w < kLatWarps; ++w) mt = fmaxf(mt, s_m[w]);
  if (sink != nullptr) mt = fmaxf(mt, sink[h]);
  float lt = sink != nullptr ? expf(sink[h] - mt) : 0.f;
  float f[kLatWarps];
#pragma unroll
  for (int w = 0; w < kLatWarps; ++w) {
    f[w] = s_m[w] == -INFINITY ? 0.f : expf(s_m[w] - mt);
    lt += s_l[w] * f[w];
  }
  const float inv = 1.f / lt;
  float* o = out + ((long long)t * H + h) * r;
  for (int c = threadIdx.x; c < r; c += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kLatWarps; ++w) v += sacc[w * r + c] * f[w];
    o[c] = v * inv;
  }
}

}  // namespace omc

using namespace omc;

extern "C" int omc_latent_kv_store(const float* dkv, long long ld, int T, int r, int dr, const void* w, int w_dt, float eps,
                                   const float* cs, int rot_dims, const int32_t* pos, const int32_t* slot,
                                   const int32_t* block_table, int max_pages, int page_size, void* pool, int pool_dt, void* stream) {
  if (dkv == nullptr || w == nullptr || cs == nullptr || pos == nullptr || slot == nullptr || block_table == nullptr || pool == nullptr ||
      T < 0 || r <= 0 || dr < 0 || rot_dims < 0 || rot_dims > dr || (rot_dims & 1) || page_size <= 0 || max_pages <= 0)
    return set_error(OMC_ERR_ARG, "omc_latent_kv_store: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(w_dt, TW, OMC_DT_SWITCH(pool_dt, TC, {
    latent_kv_store_kernel<TW, TC><<<T, 128, 0, st>>>(dkv, ld, r, dr, static_cast<const TW*>(w), eps, cs, rot_dims, pos, slot,
                                                      block_table, max_pages, page_size, static_cast<TC*>(pool));
  }))
  return check_launch("omc_latent_kv_store");
}

extern "C" int omc_latent_rope_store(const float* dkv, long long ld, int T, int r, int dr, const void* w, float eps, const float* cs,
                                     int rot_dims, const int32_t* pos, const int32_t* slot, const int32_t* block_table, int max_pages,
                                     int page_size, void* pool, const void* q, long long ldq, int H, int dn, void* qcat, int dt,
                                     void* stream) {
  if (dkv == nullptr || w == nullptr || cs == nullptr || pos == nullptr || slot == nullptr || block_table == nullptr || pool == nullptr ||
      q == nullptr || qcat == nullptr || T < 0 || r <= 0 || dr < 0 || rot_dims < 0 || rot_dims > dr || (rot_dims & 1) || page_size <= 0 ||
      max_pages <= 0 || H <= 0 || dn < 0)
    return set_error(OMC_ERR_ARG, "omc_latent_rope_store: bad argument");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(dt, TT, {
    latent_rope_store_kernel<TT><<<T, 128, 0, st>>>(dkv, ld, r, dr, static_cast<const TT*>(w), eps, cs, rot_dims, pos, slot, block_table,
                                                    max_pages, page_size, static_cast<TT*>(pool), static_cast<const TT*>(q), ldq, H, dn,
                                                    static_cast<TT*>(qcat));
  })
  return check_launch("omc_latent_rope_store");
}

extern "C" int omc_rotary_q(const void* q32, int in_dt, long long ldq, int T, int H, int dn, int dr, const float* cs, int rot_dims,
                            const int32_t* pos, void* qcat, int q_dt, int r, void* stream) {
  if (q32 == nullptr || cs == nullptr || pos == nullptr || qcat == nullptr || T < 0 || H <= 0 || dn < 0 || dr < 0 || rot_dims > dr ||
      (rot_dims & 1))
    return set_error(OMC_ERR_ARG, "omc_rotary_q: bad argument");
  if (T == 0 || dr == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMC_DT_SWITCH(in_dt, TI, OMC_DT_SWITCH(q_dt, TQ, {
    rotary_q_kernel<TI, TQ><<<T, 128, 0, st>>>(static_cast<const TI*>(q32), ldq, H, dn, dr, cs, rot_dims, pos, static_cast<TQ*>(qcat), r);
  }))
  return check_launch("omc_rotary_q");
}

extern "C" int omc_latent_attn(const void* qcat, int q_dt, int T, int H, int r, int dr, const void* pool, int pool_dt,
                               const int32_t* block_table, int max_pages, int page_size, const int32_t* pos, const int32_t* slot,
                               const float* sink, float scale, float* out, void* stream) {
  if (qcat == nullptr || pool == nullptr || block_table == nullptr || pos == nullptr || slot == nullptr || out == nullptr || T < 0 ||
      H <= 0 || r <= 0 || dr < 0 || page_size <= 0 || max_pages <= 0)
    return set_error(OMC_ERR_ARG, "omc_latent_attn: bad argument");
  if (r > 32 * kLatMaxPerLane) return set_error(OMC_ERR_SHAPE, "omc_latent_attn: latent width above 1024");
  if (H > 65535) return set_error(OMC_ERR_SHAPE, "omc_latent_attn: more than 65535 heads");
  if (T == 0) return OMC_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(float) * ((size_t)r + dr + (size_t)kLatWarps * r + 2 * kLatWarps);
  OMC_DT_SWITCH(q_dt, TQ, OMC_DT_SWITCH(pool_dt, TC, {
    latent_attn_kernel<TQ, TC><<<dim3(T, H), kLatWarps * 32, smem, st>>>(static_cast<const TQ*>(qcat), H, r, dr,
                                                                         static_cast<const TC*>(pool), block_table, max_pages,
                                                                         page_size, pos, slot, sink, scale, out);
  }))
  return check_launch("omc_latent_attn");
}

// ---------------------------------------------------------------------------------------------------------------------------
// Tensor-core kernel (bf16 storage). Rows of a tile are (token, head) pairs of one sequence portion - 64 consecutive rows of
// qcat viewed as [T * H, r + dr] - so that all heads of a token share the key tile that is staged for them; a 64-key tile
// [64][r + dr] in shared memory is the B operand of S = Q K^T as it lies (ldmatrix) and, through ldmatrix.trans over its first
// r columns, the B operand of O += P V: the cache row is read once for both. 4 row groups of 16 rows x VS warps each = 4 * VS
// warps: the VS warps of a row group split the tile's keys for the scores (row maxima and the bf16 probabilities are exchanged
// through shared memory) and the r output columns for P V (r = 512 in one warp would need 256 accumulator registers per thread;
// with VS = 4 a CTA has 16 warps to hide the latency of the dependent mma chains). Long contexts of decode rows are cut into key ranges that
// different CTAs take; their (max, sum, unnormalised output) partials are merged by latent_attn_merge_kernel, which also adds
// the sink term to the denominator.
namespace omc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

constexpr int kMmaRows = 64, kMmaKeys = 64;
constexpr int kPPitch = kMmaKeys + 8;  // row pitch of the probability tile the two warps of a row group exchange
constexpr int kMaxVS = 4;               // warps that share a row group (value columns and keys of a tile are split between them)
constexpr int kPairBytes = kMmaRows * kPPitch * 2 + kMaxVS * kMmaRows * 4;
// barrier of the VS warps (rg, rg + 4, ...) that share a row group
template <int VS>
__device__ __forceinline__ void group_sync(int rg) { asm volatile("bar.sync %0, %1;" ::"r"(rg + 1), "n"(32 * VS) : "memory"); }

struct LatMmaArgs {
  const bf16_t* q;
  const bf16_t* pool;
  const int32_t* bt;
  const int32_t* items;  // [n][8]: first_row, n_tok, slot, first_pos, key_begin, key_end, part_slot (-1: final), unused
  const float* sink;
  void* out;     // [T * H][r] fp32 or bf16
  float* ws_o;   // [part_slot][64][r]
  float* ws_ml;  // [part_slot][64][2]
  int max_pages, page_size, H, r, dr;
  float scale_log2;
  int two_buffers;  // shared memory holds two key tiles
};

__device__ __forceinline__ void st_pair(float* p, float x, float y) { *reinterpret_cast<float2*>(p) = make_float2(x, y); }
__device__ __forceinline__ void st_pair(bf16_t* p, float x, float y) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y); }

template <int VS, int NV, typename TO>  // NV: 8-column output tiles per warp; covers r <= VS * NV * 8
__global__ void __launch_bounds__(128 * VS) latent_attn_mma_kernel(LatMmaArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = a.r + a.dr, pitch = D + 8;
  bf16_t* Qs = reinterpret_cast<bf16_t*>(smem_raw);
  bf16_t* Ks = Qs + kMmaRows * pitch;
  const int32_t* it = a.items + blockIdx.x * 8;
  const int first_row = it[0], n_tok = it[1], slot = it[2], first_pos = it[3], kb = it[4], ke = it[5], part = it[6];
  const int n_rows = n_tok * a.H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, vs = warp >> 2;
  const int g = lane >> 2, t4 = lane & 3;
  const int chunks = D >> 3;  // 16-byte pieces per row
  // stage Q (rows past the portion are zero)
  {
    const bf16_t* qsrc = a.q + (long long)first_row * a.H * D;
    for (int i = tid; i < kMmaRows * chunks; i += blockDim.x) {
      const int row = i / chunks, c = i - row * chunks;
      bf16_t* dst = Qs + row * pitch + c * 8;
      if (row < n_rows) cp_async16(smem_u32(dst), qsrc + (long long)row * D + c * 8);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
  const int row0 = rg * 16 + g, row1 = row0 + 8;
  // last key (inclusive) each of this thread's two rows may see
  const int lim0 = row0 < n_rows ? first_pos + row0 / a.H : -1;
  const int lim1 = row1 < n_rows ? first_pos + row1 / a.H : -1;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  const int nv = a.r >> 3;                       // output tiles in total
  const int nv_per = (nv + VS - 1) / VS;         // this warp's share: tiles [vs * nv_per, min(nv, (vs + 1) * nv_per))
  const int nv0 = vs * nv_per;
  const int32_t* bt = a.bt + (long long)slot * a.max_pages;
  const int k_end = min(ke, first_pos + n_tok);  // exclusive
  // key tiles: with two buffers the next tile is on its way while this one is computed
  auto stage_keys = [&](bf16_t* buf, int j0) {
    for (int i = tid; i < kMmaKeys * chunks; i += blockDim.x) {
      const int key = i / chunks, c = i - key * chunks;
      bf16_t* dst = buf + key * pitch + c * 8;
      const int j = j0 + key;
      if (j < k_end) {
        const bf16_t* src = a.pool + ((long long)bt[j / a.page_size] * a.page_size + j % a.page_size) * D + c * 8;
        cp_async16(smem_u32(dst), src);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  bf16_t* Kbuf[2] = {Ks, a.two_buffers ? Ks + kMmaKeys * pitch : Ks};
  constexpr int NS = 8 / VS;                 // 8-key score tiles per warp
  const int kofs = vs * (kMmaKeys / VS);     // first key of this warp's share of a tile
  bf16_t* Ps = Ks + (a.two_buffers ? 2 : 1) * kMmaKeys * pitch;       // [64][kPPitch] probabilities (VS > 1 only)
  float* s_x = reinterpret_cast<float*>(Ps + kMmaRows * kPPitch);     // [VS][64] row maxima / sums of the warps of a row group
  if (kb < k_end) stage_keys(Kbuf[0], kb);
  int kt = 0;
  for (int j0 = kb; j0 < k_end; j0 += kMmaKeys, ++kt) {
    bf16_t* Kc = Kbuf[kt & 1];
    if (a.two_buffers) {
      if (j0 + kMmaKeys < k_end) {
        stage_keys(Kbuf[(kt + 1) & 1], j0 + kMmaKeys);  // that buffer was released by the barrier that ended the previous tile
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        cp_async_wait_all();
      }
    } else {
      if (kt > 0) stage_keys(Kc, j0);
      cp_async_wait_all();
    }
    __syncthreads();
    if (rg * 16 < n_rows) {  // a row group without rows (decode: H rows of the 64) only helps staging the tiles
    // S = Q K^T for this warp's 16 rows x its keys: all 64 keys, or with two warps per row group the half [vs * 32, vs * 32 + 32)
    // (the partner computes the other half; the row maximum and the probabilities are exchanged through shared memory)
    float s[NS][4], s2[NS][4];  // two accumulator sets over alternating K slices: twice the independent mma chains per warp
#pragma unroll
    for (int n = 0; n < NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = s2[n][0] = s2[n][1] = s2[n][2] = s2[n][3] = 0.f;
    const uint32_t q_base = smem_u32(Qs + (rg * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * pitch + 8 * (lane >> 4));
    const uint32_t k_base = smem_u32(Kc + (kofs + (lane & 7) + 8 * (lane >> 4)) * pitch + 8 * ((lane >> 3) & 1));
#pragma unroll 2
    for (int kk = 0; kk < D; kk += 32) {
      uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
      ldsm_x4(q_base + kk * 2, a0, a1, a2, a3);
      const bool second = kk + 16 < D;  // D is a multiple of 16, not always of 32
      if (second) ldsm_x4(q_base + (kk + 16) * 2, c0, c1, c2, c3);
#pragma unroll
      for (int n2 = 0; n2 < NS / 2; ++n2) {  // key blocks of 16
        uint32_t b0, b1, b2, b3;
        ldsm_x4(k_base + (n2 * 16 * pitch + kk) * 2, b0, b1, b2, b3);
        mma_bf16(s[2 * n2], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[2 * n2 + 1], a0, a1, a2, a3, b2, b3);
        if (second) {
          ldsm_x4(k_base + (n2 * 16 * pitch + kk + 16) * 2, b0, b1, b2, b3);
          mma_bf16(s2[2 * n2], c0, c1, c2, c3, b0, b1);
          mma_bf16(s2[2 * n2 + 1], c0, c1, c2, c3, b2, b3);
        }
      }
    }
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      s[n][0] += s2[n][0];
      s[n][1] += s2[n][1];
      s[n][2] += s2[n][2];
      s[n][3] += s2[n][3];
    }
    // mask + online softmax (base-2 exponent, scale folded in)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const int key = j0 + kofs + n * 8 + 2 * t4;
      s[n][0] = key <= lim0 ? s[n][0] * a.scale_log2 : -INFINITY;
      s[n][1] = key + 1 <= lim0 ? s[n][1] * a.scale_log2 : -INFINITY;
      s[n][2] = key <= lim1 ? s[n][2] * a.scale_log2 : -INFINITY;
      s[n][3] = key + 1 <= lim1 ? s[n][3] * a.scale_log2 : -INFINITY;
      mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
      mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if constexpr (VS > 1) {
      if (t4 == 0) {
        s_x[vs * kMmaRows + row0] = mx0;
        s_x[vs * kMmaRows + row1] = mx1;
      }
      group_sync<VS>(rg);
#pragma unroll
      for (int v = 0; v < VS; ++v) {
        mx0 = fmaxf(mx0, s_x[v * kMmaRows + row0]);
        mx1 = fmaxf(mx1, s_x[v * kMmaRows + row1]);
      }
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;  // rows that see nothing yet
    const float c0 = exp2f(m0 - ms0), c1 = exp2f(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t p[NS][2];
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const float e0 = exp2f(s[n][0] - ms0), e1 = exp2f(s[n][1] - ms0), e2 = exp2f(s[n][2] - ms1), e3 = exp2f(s[n][3] - ms1);
      p[n][0] = pack2_bf16(e0, e1);
      p[n][1] = pack2_bf16(e2, e3);
      // the denominator sums the ROUNDED probabilities, the ones the numerator uses
      const float2 f0 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&p[n][0]));
      const float2 f1 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&p[n][1]));
      rs0 += f0.x + f0.y;
      rs1 += f1.x + f1.y;
    }
    l0 = l0 * c0 + rs0;  // with two warps per row group: the sum over this warp's keys only, completed after the last tile
    l1 = l1 * c1 + rs1;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      o[j][0] *= c0;
      o[j][1] *= c0;
      o[j][2] *= c1;
      o[j][3] *= c1;
    }
    if constexpr (VS > 1) {
#pragma unroll
      for (int n = 0; n < NS; ++n) {
        *reinterpret_cast<uint32_t*>(Ps + row0 * kPPitch + kofs + n * 8 + 2 * t4) = p[n][0];
        *reinterpret_cast<uint32_t*>(Ps + row1 * kPPitch + kofs + n * 8 + 2 * t4) = p[n][1];
      }
      group_sync<VS>(rg);
    }
    // O += P V over this warp's output tiles (pairs of 8-column tiles per ldmatrix.x4.trans)
    const uint32_t v_base = smem_u32(Kc + ((lane & 7) + 8 * ((lane >> 3) & 1)) * pitch + 8 * (lane >> 4));
    const uint32_t p_base = smem_u32(Ps + (rg * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * kPPitch + 8 * (lane >> 4));
#pragma unroll
    for (int kb16 = 0; kb16 < 4; ++kb16) {
      uint32_t a0, a1, a2, a3;
      if constexpr (VS > 1) {
        ldsm_x4(p_base + kb16 * 16 * 2, a0, a1, a2, a3);
      } else {
        a0 = p[(2 * kb16) % NS][0], a1 = p[(2 * kb16) % NS][1], a2 = p[(2 * kb16 + 1) % NS][0], a3 = p[(2 * kb16 + 1) % NS][1];
      }
#pragma unroll
      for (int j = 0; j < NV; j += 2) {
        const int tile = nv0 + j;
        if (j < nv_per && tile < nv) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(v_base + (kb16 * 16 * pitch + tile * 8) * 2, b0, b1, b2, b3);
          mma_bf16(o[j], a0, a1, a2, a3, b0, b1);
          if (j + 1 < nv_per && tile + 1 < nv) mma_bf16(o[j + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    }
    __syncthreads();  // every warp is done with this tile's buffer
  }
  // row sums over the quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if constexpr (VS > 1) {  // the other warps' shares of the denominator
    __syncthreads();
    if (t4 == 0) {
      s_x[vs * kMmaRows + row0] = l0;
      s_x[vs * kMmaRows + row1] = l1;
    }
    __syncthreads();
    l0 = l1 = 0.f;
#pragma unroll
    for (int v = 0; v < VS; ++v) {
      l0 += s_x[v * kMmaRows + row0];
      l1 += s_x[v * kMmaRows + row1];
    }
  }
  if (part < 0) {
    float d0 = l0, d1 = l1;
    if (a.sink != nullptr) {
      if (row0 < n_rows) d0 += exp2f(a.sink[row0 % a.H] * 1.4426950408889634f - m0);
      if (row1 < n_rows) d1 += exp2f(a.sink[row1 % a.H] * 1.4426950408889634f - m1);
    }
    const float i0 = 1.f / d0, i1 = 1.f / d1;
    TO* out0 = static_cast<TO*>(a.out) + ((long long)first_row * a.H + row0) * a.r;
    TO* out1 = static_cast<TO*>(a.out) + ((long long)first_row * a.H + row1) * a.r;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int tile = nv0 + j;
      if (j < nv_per && tile < nv) {
        const int col = tile * 8 + 2 * t4;
        if (row0 < n_rows) st_pair(out0 + col, o[j][0] * i0, o[j][1] * i0);
        if (row1 < n_rows) st_pair(out1 + col, o[j][2] * i1, o[j][3] * i1);
      }
    }
  } else {
    float* wo = a.ws_o + (long long)part * kMmaRows * a.r;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int tile = nv0 + j;
      if (j < nv_per && tile < nv) {
        const int col = tile * 8 + 2 * t4;
        *reinterpret_cast<float2*>(wo + (long long)row0 * a.r + col) = make_float2(o[j][0], o[j][1]);
        *reinterpret_cast<float2*>(wo + (long long)row1 * a.r + col) = make_float2(o[j][2], o[j][3]);
      }
    }
    if (vs == 0 && t4 == 0) {
      float* ml = a.ws_ml + (long long)part * kMmaRows * 2;
      ml[row0 * 2] = m0;
      ml[row0 * 2 + 1] = l0;
      ml[row1 * 2] = m1;
      ml[row1 * 2 + 1] = l1;
    }
  }
}

// merges[i] = (first q row = first_row * H, n_rows, first part slot, n_parts): one CTA per (group, row), threads over columns,
// four parts' loads in flight per thread (a warp that walked parts and columns one load at a time spent 70 us on latency).
constexpr int kMergeMaxParts = 64;
template <typename TO>
__global__ void __launch_bounds__(128) latent_attn_merge_kernel(const int32_t* __restrict__ merges, const float* __restrict__ ws_o,
                                                                const float* __restrict__ ws_ml, const float* __restrict__ sink, int H,
                                                                int r, TO* __restrict__ out) {
  __shared__ float s_f[kMergeMaxParts];
  __shared__ float s_inv;
  const int32_t* mg = merges + blockIdx.x * 4;
  const int qrow0 = mg[0], n_rows = mg[1], part0 = mg[2], n_parts = mg[3];
  const int row = blockIdx.y;
  if (row >= n_rows) return;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float mt = -INFINITY;
    for (int p = lane; p < n_parts; p += 32) mt = fmaxf(mt, ws_ml[((long long)(part0 + p) * kMmaRows + row) * 2]);
    mt = seq_warp_max(mt);
    const float sk = sink != nullptr ? sink[(qrow0 + row) % H] * 1.4426950408889634f : -INFINITY;
    mt = fmaxf(mt, sk);
    float den = 0.f;
    for (int p = lane; p < n_parts; p += 32) {
      const float* ml = ws_ml + ((long long)(part0 + p) * kMmaRows + row) * 2;
      const float f = ml[0] == -INFINITY ? 0.f : exp2f(ml[0] - mt);
      s_f[p] = f;
      den += ml[1] * f;
    }
    den = seq_warp_sum(den);
    if (sink != nullptr) den += exp2f(sk - mt);
    if (lane == 0) s_inv = 1.f / den;
  }
  __syncthreads();
  const float inv = s_inv;
  const float* base = ws_o + ((long long)part0 * kMmaRows + row) * r;
  const long long ps = (long long)kMmaRows * r;  // stride between parts
  for (int c = threadIdx.x; c < r; c += blockDim.x) {
    float v = 0.f;
    int p = 0;
    for (; p + 4 <= n_parts; p += 4) {
      const float a0 = base[p * ps + c], a1 = base[(p + 1) * ps + c], a2 = base[(p + 2) * ps + c], a3 = base[(p + 3) * ps + c];
      v = fmaf(a0, s_f[p], v);
      v = fmaf(a1, s_f[p + 1], v);
      v = fmaf(a2, s_f[p + 2], v);
      v = fmaf(a3, s_f[p + 3], v);
    }
    for (; p < n_parts; ++p) v = fmaf(base[p * ps + c], s_f[p], v);
    stf(out + ((long long)qrow0 + row) * r + c, v * inv);
  }
}

// Work list of a decode-only step written on the device (so that the step can be replayed from a CUDA graph while the contexts
// grow): row b at position pos[b] sees pos[b] + 1 keys, cut into `parts` ranges of whole 64-key tiles (ranges past the end stay
// empty and contribute nothing to the merge).
__global__ void latent_decode_items_kernel(const int32_t* __restrict__ pos, const int32_t* __restrict__ slot, int B, int H, int parts,
                                           int32_t* __restrict__ items, int32_t* __restrict__ merges) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * parts) return;
  const int b = i / parts, j = i - b * parts;
  const int keys = pos[b] + 1;
  const int span = ((keys + parts - 1) / parts + kMmaKeys - 1) / kMmaKeys * kMmaKeys;
  int32_t* it = items + (long long)i * 8;
  it[0] = b;
  it[1] = 1;
  it[2] = slot[b];
  it[3] = pos[b];
  it[4] = min(j * span, keys);
  it[5] = min((j + 1) * span, keys);
  it[6] = parts > 1 ? i : -1;
  it[7] = 0;
  if (j == 0 && parts > 1) {
    int32_t* mg = merges + b * 4;
    mg[0] = b * H;
    mg[1] = H;
    mg[2] = b * parts;
    mg[3] = parts;
  }
}

template <int VS, int NV, typename TO>
static int launch_lat_mma_t(const LatMmaArgs& a, int n_items, size_t smem, cudaStream_t st) {
  static bool attr_done[kMaxDevices] = {};
  const int dev = cur_device();
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(latent_attn_mma_kernel<VS, NV, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return set_error(OMC_ERR_CUDA, cudaGetErrorString(e));
    attr_done[dev] = true;
  }
  latent_attn_mma_kernel<VS, NV, TO><<<n_items, 128 * VS, smem, st>>>(a);
  return check_launch("omc_latent_attn_mma");
}

template <int VS, int NV>
static int launch_lat_mma(const LatMmaArgs& a, int out_dt, int n_items, size_t smem, cudaStream_t st) {
  if (out_dt == OMC_DT_BF16) return launch_lat_mma_t<VS, NV, bf16_t>(a, n_items, smem, st);
  return launch_lat_mma_t<VS, NV, float>(a, n_items, smem, st);
}

}  // namespace omc

extern "C" int omc_latent_attn_mma(const void* qcat, int T, int H, int r, int dr, const void* pool, const int32_t* block_table,
                                   int max_pages, int page_size, const int32_t* items, int n_items, const int32_t* merges,
                                   int n_merges, const float* sink, float scale, void* out, int out_dt, float* ws_o, float* ws_ml,
                                   void* stream) {
  if (qcat == nullptr || pool == nullptr || block_table == nullptr || items == nullptr || out == nullptr || T < 0 || H <= 0 ||
      page_size <= 0 || max_pages <= 0 || n_items < 0 || n_merges < 0 || (n_merges > 0 && (merges == nullptr || ws_o == nullptr || ws_ml == nullptr)))
    return set_error(OMC_ERR_ARG, "omc_latent_attn_mma: bad argument");
  if (r <= 0 || r % 16 != 0 || r > 512 || dr < 0 || dr % 16 != 0 || H > kMmaRows)
    return set_error(OMC_ERR_SHAPE, "omc_latent_attn_mma: latent width a multiple of 16 up to 512, rotated width a multiple of 16, at most 64 heads");
  if (n_items == 0) return OMC_OK;
  const int D = r + dr;
  const size_t extra = r > 128 ? kPairBytes : 0;  // several warps per row group exchange probabilities
  size_t smem = (size_t)(kMmaRows + 2 * kMmaKeys) * (D + 8) * sizeof(bf16_t) + extra;
  int two = 1;
  if (smem > 227 * 1024) {
    two = 0;
    smem = (size_t)(kMmaRows + kMmaKeys) * (D + 8) * sizeof(bf16_t) + extra;
  }
  if (smem > 227 * 1024) return set_error(OMC_ERR_SHAPE, "omc_latent_attn_mma: rows too wide for shared memory");
  LatMmaArgs a{static_cast<const bf16_t*>(qcat), static_cast<const bf16_t*>(pool), block_table, items, sink, out, ws_o, ws_ml,
               max_pages, page_size, H, r, dr, scale * 1.4426950408889634f, two};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  if (out_dt != OMC_DT_F32 && out_dt != OMC_DT_BF16) return set_error(OMC_ERR_ARG, "omc_latent_attn_mma: unknown output dtype");
  if (r <= 64) rc = launch_lat_mma<1, 8>(a, out_dt, n_items, smem, st);
  else if (r <= 128) rc = launch_lat_mma<1, 16>(a, out_dt, n_items, smem, st);
  else if (r <= 256) rc = launch_lat_mma<2, 16>(a, out_dt, n_items, smem, st);
  else rc = launch_lat_mma<4, 16>(a, out_dt, n_items, smem, st);  // 16 warps: four per row group, 128 value columns and 16 keys each
  if (rc != OMC_OK || n_merges == 0) return rc;
  if (out_dt == OMC_DT_BF16)
    latent_attn_merge_kernel<bf16_t><<<dim3(n_merges, kMmaRows), 128, 0, st>>>(merges, ws_o, ws_ml, sink, H, r, static_cast<bf16_t*>(out));
  else
    latent_attn_merge_kernel<float><<<dim3(n_merges, kMmaRows), 128, 0, st>>>(merges, ws_o, ws_ml, sink, H, r, static_cast<float*>(out));
  return check_launch("omc_latent_attn_merge");
}

extern "C" int omc_latent_decode_items(const int32_t* pos, const int32_t* slot, int B, int H, int parts, int32_t* items, int32_t* merges,
                                       void* stream) {
  if (pos == nullptr || slot == nullptr || items == nullptr || B < 0 || H <= 0 || parts <= 0 || parts > kMergeMaxParts ||
      (parts > 1 && merges == nullptr))
    return set_error(OMC_ERR_ARG, "omc_latent_decode_items: bad argument");
  if (B == 0) return OMC_OK;
  const int n = B * parts;
  latent_decode_items_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(pos, slot, B, H, parts, items, merges);
  return check_launch("omc_latent_decode_items");
}
