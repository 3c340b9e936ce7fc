// Strided batched GEMM on the CUDA cores, fp32 accumulation, any shape and alignment.
//
//   out(t, h, n) = epilogue( sum_k x(t, h, k) * w(h, k, n) )      t < M, h < H, n < N, k < K
//   x(t, h, k)   = x  [t * ldx + h * sxh + k]
//   w(h, k, n)   = w  [h * swh + k * swk + n * swn]
//   out(t, h, n) = out[t * ldo + h * soh + n]
//
// Three users:
//   * true 32-bit linear layers (T = float; the tcgen05 GEMM takes 16-bit operands only), and 16-bit linear
//     layers whose K or base address misses the 16-byte rule of the TMA path: H = 1, swk = 1, swn = ldw;
//   * the per-head products of latent attention: q_h -> W_uk,h^T q_h (swk = rank, swn = 1) and
//     o_h -> W_uv,h o_h (swk = 1, swn = rank), optionally scaled per (token, head) by an output gate.
// 64 x 64 output tile per CTA, 16-deep k slices through shared memory, 4 x 4 outputs per thread.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

struct BgArgs {
  const void* x; int64_t ldx, sxh;
  const void* w; int64_t swh, swk, swn;
  const void* bias;              // [N] of T, h-independent, or null
  const float* row_scale; int64_t lds;   // scale(t, h) = row_scale[t * lds + h], or null
  void* out; int64_t ldo, soh;
  int M, N, K, H, act, act_start;
};

__device__ __forceinline__ float act_sq(float x, int act) {
  if (act == LLMSS_ACT_RELU2) { const float r = fmaxf(x, 0.f); return r * r; }
  return act_apply(x, act);
}

template <typename T, bool OUT_F32>
__global__ void __launch_bounds__(NT) bgemm_kernel(BgArgs a) {
  __shared__ float Xs[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int h = blockIdx.z;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const T* x = reinterpret_cast<const T*>(a.x) + (int64_t)h * a.sxh;
  const T* w = reinterpret_cast<const T*>(a.w) + (int64_t)h * a.swh;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const bool n_fast = (a.swn == 1);
  for (int k0 = 0; k0 < a.K; k0 += BK) {
    for (int idx = threadIdx.x; idx < BM * BK; idx += NT) {
      const int m = idx / BK, k = idx % BK;
      float v = 0.f;
      if (m0 + m < a.M && k0 + k < a.K) v = to_f32(x[(int64_t)(m0 + m) * a.ldx + k0 + k]);
      Xs[k][m] = v;
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += NT) {
      int n, k;
      if (n_fast) { k = idx / BN; n = idx % BN; } else { n = idx / BK; k = idx % BK; }
      float v = 0.f;
      if (n0 + n < a.N && k0 + k < a.K) v = to_f32(w[(int64_t)(k0 + k) * a.swk + (int64_t)(n0 + n) * a.swn]);
      Ws[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = Xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  using TO = typename std::conditional<OUT_F32, float, T>::type;
  TO* out = reinterpret_cast<TO*>(a.out) + (int64_t)h * a.soh;
  const T* bias = reinterpret_cast<const T*>(a.bias);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= a.M) continue;
    const float rs = a.row_scale != nullptr ? a.row_scale[(int64_t)m * a.lds + h] : 1.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= a.N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += to_f32(bias[n]);
      if (a.act != LLMSS_ACT_NONE && n >= a.act_start) v = act_sq(v, a.act);
      out[(int64_t)m * a.ldo + n] = from_f32<TO>(v * rs);
    }
  }
}

template <typename T>
int launch_bg(const BgArgs& a, int out_f32, cudaStream_t stream) {
  dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM, a.H);
  if (out_f32) bgemm_kernel<T, true><<<grid, NT, 0, stream>>>(a);
  else bgemm_kernel<T, false><<<grid, NT, 0, stream>>>(a);
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace

LLMSS_API int llmss_bgemm_simt(const void* x, int64_t ldx, int64_t sxh, const void* w, int64_t swh, int64_t swk,
                               int64_t swn, const void* bias, const float* row_scale, int64_t lds, void* out,
                               int64_t ldo, int64_t soh, int M, int N, int K, int H, int act, int act_start,
                               int dtype, int out_f32, cudaStream_t stream) {
  LLMSS_REQUIRE(M >= 0 && N > 0 && K > 0 && H > 0 && H <= 65535, "bgemm_simt: bad shape M=%d N=%d K=%d H=%d", M, N, K, H);
  LLMSS_REQUIRE((M + BM - 1) / BM <= 65535, "bgemm_simt: M=%d too large", M);
  if (M == 0) return 0;
  BgArgs a{x, ldx, sxh, w, swh, swk, swn, bias, row_scale, lds, out, ldo, soh, M, N, K, H, act, act_start};
  if (dtype == LLMSS_F32) return launch_bg<float>(a, 1, stream);
  if (dtype == LLMSS_BF16) return launch_bg<__nv_bfloat16>(a, out_f32, stream);
  if (dtype == LLMSS_F16) return launch_bg<__half>(a, out_f32, stream);
  LLMSS_REQUIRE(false, "bgemm_simt: bad dtype %d", dtype);
}
