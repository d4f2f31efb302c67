// Linear layer for any shape and for fp32 as well as bf16 storage: Y = act(alpha * X W^T), fp32 accumulation on the FMA pipe.
//
// This is the kernel a new decoder is brought up on, the true-fp32 path of the sequence-step models (no reduced-precision
// matrix mode anywhere), and the path for shapes the tcgen05 GEMM does not take (dimensions that are not multiples of 8, head
// slices of a few dozen columns). 64 x 64 output tile per CTA, 256 threads with 4 x 4 outputs each, K walked in slices of 16
// through shared memory (operands converted to fp32 when they are staged). blockIdx.z walks a batch of independent problems
// that are column slices of the same buffers (attention heads); an optional tile -> group table turns it into the grouped
// product of expert-sorted rows. Each output accumulates its K terms in ascending order, whatever the M of the call.
#include "seq_common.cuh"

namespace omc {

constexpr int kLinBM = 64, kLinBN = 64, kLinBK = 16;

struct LinearArgs {
  const void* X;
  const void* W;
  void* Y;
  long long ldx, sx, ldw, sw, ldy, sy, group_stride;
  const int32_t* tile_group;
  int M, N, K;
  float alpha;
  int act;
};

__device__ __forceinline__ float apply_act(float z, int act) {
  if (act == OMC_ACT_RELU2) {
    z = fmaxf(z, 0.f);
    return z * z;
  }
  if (act == OMC_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z;
}

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256) linear_tile_kernel(LinearArgs a) {
  __shared__ float xs[kLinBK][kLinBM + 4];
  __shared__ float ws[kLinBK][kLinBN + 4];
  const int m0 = blockIdx.y * kLinBM, n0 = blockIdx.x * kLinBN;
  const TX* X = static_cast<const TX*>(a.X) + (long long)blockIdx.z * a.sx;
  const TW* W = static_cast<const TW*>(a.W) + (long long)blockIdx.z * a.sw;
  TY* Y = static_cast<TY*>(a.Y) + (long long)blockIdx.z * a.sy;
  if (a.tile_group != nullptr) {
    const int g = a.tile_group[blockIdx.y];
    if (g < 0) return;
    W += (long long)g * a.group_stride;
  }
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  // staging: thread -> (row = tid / 4, k quarter = tid % 4): 4 consecutive k of one row
  const int lr = threadIdx.x >> 2, lk = (threadIdx.x & 3) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < a.K; k0 += kLinBK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int m = m0 + lr, n = n0 + lr;
      xs[lk + j][lr] = (m < a.M && k < a.K) ? ldf(X + (long long)m * a.ldx + k) : 0.f;
      ws[lk + j][lr] = (n < a.N && k < a.K) ? ldf(W + (long long)n * a.ldw + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kLinBK; ++k) {
      const float4 xv = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float xr[4] = {xv.x, xv.y, xv.z, xv.w}, wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xr[i], wr[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < a.N) stf(Y + (long long)m * a.ldy + n, apply_act(acc[i][j] * a.alpha, a.act));
    }
  }
}

template <typename TX, typename TW>
static int launch_linear(const LinearArgs& a, int y_dt, int batch, cudaStream_t st) {
  dim3 grid((a.N + kLinBN - 1) / kLinBN, (a.M + kLinBM - 1) / kLinBM, batch);
  if (y_dt == OMC_DT_F32) linear_tile_kernel<TX, TW, float><<<grid, 256, 0, st>>>(a);
  else if (y_dt == OMC_DT_BF16) linear_tile_kernel<TX, TW, bf16_t><<<grid, 256, 0, st>>>(a);
  else return set_error(OMC_ERR_ARG, "omc_linear: unknown output dtype");
  return check_launch("omc_linear");
}

}  // namespace omc

extern "C" int omc_linear(const void* X, int x_dt, long long ldx, long long sx, const void* W, int w_dt, long long ldw,
                          long long sw, void* Y, int y_dt, long long ldy, long long sy, int M, int N, int K, int batch,
                          float alpha, int act, const int32_t* tile_group, long long group_stride, void* stream) {
  using namespace omc;
  if (X == nullptr || W == nullptr || Y == nullptr || N <= 0 || K <= 0 || M < 0 || batch <= 0)
    return set_error(OMC_ERR_ARG, "omc_linear: bad argument");
  if (M == 0) return OMC_OK;
  if (tile_group != nullptr && batch != 1) return set_error(OMC_ERR_ARG, "omc_linear: a tile table excludes a batch");
  if ((long long)((M + kLinBM - 1) / kLinBM) > 65535 || batch > 65535)
    return set_error(OMC_ERR_SHAPE, "omc_linear: more than 65535 row tiles or batch items");
  LinearArgs a{X, W, Y, ldx, sx, ldw, sw, ldy, sy, group_stride, tile_group, M, N, K, alpha, act};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (x_dt == OMC_DT_F32 && w_dt == OMC_DT_F32) return launch_linear<float, float>(a, y_dt, batch, st);
  if (x_dt == OMC_DT_F32 && w_dt == OMC_DT_BF16) return launch_linear<float, bf16_t>(a, y_dt, batch, st);
  if (x_dt == OMC_DT_BF16 && w_dt == OMC_DT_BF16) return launch_linear<bf16_t, bf16_t>(a, y_dt, batch, st);
  return set_error(OMC_ERR_ARG, "omc_linear: operand dtypes must be (f32, f32), (f32, bf16) or (bf16, bf16)");
}
