// Grouped-query softmax attention with separate key / value sizes, per-head query / key norm, a query temperature and a
// learned distance bias, over the paged cache -- the generic (any head size, 16- or 32-bit) form.
//
//   qknorm_kv_write : per token and head, rms_div(q) * q_w (times the query temperature 1 + coef * ln(floor((p + 1) /
//                     every) + 1)) -> queries in the compute type; rms_div(k) * k_w -> key page; v -> value page.  The
//                     counterpart of rope_kv_write for a design whose positions enter through distances, not rotations.
//   attention_bias  : out_ih = gate_ih * sum_j softmax_j(scale * q_ih . k_jg + bias[h][min(i - j, last)]) v_jg ,  j <= i.
//                     One CTA = one sequence x one key/value head x up to 8 (query row, query head of the group) pairs;
//                     its warps share every 32-key tile of K and V, staged once in shared memory in 32-bit.  A warp owns
//                     one pair: lane = key inside the tile for the scores, lane = output channel (mod 32) for P V.
//                     Scores, softmax and accumulation are 32-bit with full-precision exponentials.
// Page layouts: keys [num_blocks, kv_heads, block_size, dk], values [num_blocks, kv_heads, block_size, dv].
#include "common.cuh"

namespace {

constexpr int NW = 8, TK = 32, MAXV = 8;   // warps per CTA, keys per tile, output channels per lane (dv <= 256)

template <typename T>
__global__ void __launch_bounds__(256) qknorm_kv_write_kernel(const float* __restrict__ qkv, int64_t ld, int hq, int hkv, int dk,
                                                              int dv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                                              float eps, float coef, int every, const int* __restrict__ positions,
                                                              const int* __restrict__ slots, T* __restrict__ k_cache,
                                                              T* __restrict__ v_cache, int bs, T* __restrict__ q_out, int T_) {
  const int nh = hq + 2 * hkv;
  const int64_t unit = (int64_t)blockIdx.x * NW + (threadIdx.x >> 5);
  if (unit >= (int64_t)T_ * nh) return;
  const int64_t t = unit / nh;
  const int h = (int)(unit % nh), lane = threadIdx.x & 31;
  const float* row = qkv + t * ld;
  const int slot = slots[t];
  if (h < hq + hkv) {
    const float* x = row + (int64_t)h * dk;
    float ss = 0.f;
    for (int c = lane; c < dk; c += 32) ss = fmaf(x[c], x[c], ss);
    float r = rsqrtf(warp_sum(ss) / dk + eps);
    if (h < hq) {
      if (coef != 0.f) r *= 1.f + coef * logf((float)((positions[t] + 1) / every) + 1.f);
      for (int c = lane; c < dk; c += 32) q_out[t * hq * dk + (int64_t)h * dk + c] = from_f32<T>(x[c] * r * q_w[c]);
    } else if (slot >= 0) {
      T* dst = k_cache + (((int64_t)(slot / bs) * hkv + (h - hq)) * bs + slot % bs) * dk;
      for (int c = lane; c < dk; c += 32) dst[c] = from_f32<T>(x[c] * r * k_w[c]);
    }
  } else if (slot >= 0) {
    const int g = h - hq - hkv;
    const float* x = row + (int64_t)(hq + hkv) * dk + (int64_t)g * dv;
    T* dst = v_cache + (((int64_t)(slot / bs) * hkv + g) * bs + slot % bs) * dv;
    for (int c = lane; c < dv; c += 32) dst[c] = from_f32<T>(x[c]);
  }
}

// x[t, h * dv + c] *= sigmoid(gate[t, h]) in place: the output gate behind an attention kernel that has no gate of its own
template <typename T>
__global__ void __launch_bounds__(256) head_gate_kernel(T* __restrict__ x, int64_t ldx, const float* __restrict__ gate, int64_t ldg,
                                                        int hq, int dv) {
  const int64_t t = blockIdx.x;
  for (int c = threadIdx.x; c < hq * dv; c += 256) {
    const float g = 1.f / (1.f + expf(-gate[t * ldg + c / dv]));
    x[t * ldx + c] = from_f32<T>(to_f32(x[t * ldx + c]) * g);
  }
}

struct AbArgs {
  const void* q; int64_t ldq;
  const void* k_cache; const void* v_cache;
  const int* block_tables; int max_blocks, bs;
  const int* seq_lens; const int* cu_q;
  const float* bias; int n_dist;          // [hq][n_dist]
  const float* gate; int64_t ldg;         // [T][hq] logits, or null
  void* out;                              // [T][hq * dv]
  int hq, hkv, dk, dv, nh, rows, hsub;    // nh: query heads per CTA; rows: query rows per CTA; hsub: CTAs per kv head
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(NW * 32) attention_bias_kernel(AbArgs a) {
  extern __shared__ float sm[];
  const int b = blockIdx.z;
  const int q0 = a.cu_q[b], ql = a.cu_q[b + 1] - q0, L = a.seq_lens[b];
  const int r0 = blockIdx.x * a.rows;
  if (r0 >= ql || L <= 0) return;
  const int g = blockIdx.y / a.hsub, hs = blockIdx.y % a.hsub;
  const int gsz = a.hq / a.hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dk = a.dk, dv = a.dv, dkp = dk + 1;
  float* qs = sm;                      // [NW][dk]
  float* ks = qs + NW * dk;            // [TK][dk + 1]
  float* vs = ks + TK * dkp;           // [TK][dv]
  // this warp's (row, head)
  const int hl = warp % a.nh, rl = warp / a.nh;
  const int hin = hs * NW + hl;                 // head inside the group
  const int row = r0 + rl;
  const bool active = rl < a.rows && row < ql && hin < gsz;
  const int h = g * gsz + hin;
  const int ctx = L - ql;
  const int qpos = ctx + row;                   // absolute position of the query
  const T* qg = reinterpret_cast<const T*>(a.q);
  if (active)
    for (int c = lane; c < dk; c += 32) qs[warp * dk + c] = to_f32(qg[(int64_t)(q0 + row) * a.ldq + (int64_t)h * dk + c]) * a.scale;
  const int last_row = min(ql, r0 + a.rows) - 1;
  const int kend = ctx + last_row + 1;          // keys 0 .. kend - 1 are visible to some row of this CTA
  float m = -INFINITY, l = 0.f, acc[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) acc[i] = 0.f;
  const T* kc = reinterpret_cast<const T*>(a.k_cache);
  const T* vc = reinterpret_cast<const T*>(a.v_cache);
  const float* brow = a.bias != nullptr ? a.bias + (int64_t)(active ? h : 0) * a.n_dist : nullptr;
  for (int k0 = 0; k0 < kend; k0 += TK) {
    const int nk = min(TK, kend - k0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nk * dk; idx += NW * 32) {
      const int kk = idx / dk, c = idx % dk, pos = k0 + kk;
      const int blk = a.block_tables[(int64_t)b * a.max_blocks + pos / a.bs];
      ks[kk * dkp + c] = to_f32(kc[(((int64_t)blk * a.hkv + g) * a.bs + pos % a.bs) * dk + c]);
    }
    for (int idx = threadIdx.x; idx < nk * dv; idx += NW * 32) {
      const int kk = idx / dv, c = idx % dv, pos = k0 + kk;
      const int blk = a.block_tables[(int64_t)b * a.max_blocks + pos / a.bs];
      vs[kk * dv + c] = to_f32(vc[(((int64_t)blk * a.hkv + g) * a.bs + pos % a.bs) * dv + c]);
    }
    __syncthreads();
    if (!active || k0 > qpos) continue;
    const int kpos = k0 + lane;
    float sc = -INFINITY;
    if (lane < nk && kpos <= qpos) {
      float d = 0.f;
      const float* kr = ks + lane * dkp;
      const float* qr = qs + warp * dk;
      for (int c = 0; c < dk; ++c) d = fmaf(qr[c], kr[c], d);
      sc = d;
      if (brow != nullptr) sc += brow[min(qpos - kpos, a.n_dist - 1)];
    }
    const float mt = warp_max(sc);
    const float mn = fmaxf(m, mt);
    const float corr = expf(m - mn);            // m = -inf on the first tile: 0
    const float p = sc == -INFINITY ? 0.f : expf(sc - mn);
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) acc[i] *= corr;
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      if (pk == 0.f) continue;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) acc[i] = fmaf(pk, vs[kk * dv + c], acc[i]);
      }
    }
  }
  if (!active) return;
  float gsc = 1.f / l;
  if (a.gate != nullptr) gsc *= 1.f / (1.f + expf(-a.gate[(int64_t)(q0 + row) * a.ldg + h]));
  T* og = reinterpret_cast<T*>(a.out) + (int64_t)(q0 + row) * a.hq * dv + (int64_t)h * dv;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) og[c] = from_f32<T>(acc[i] * gsc);
  }
}

}  // namespace

LLMSS_API int llmss_qknorm_kv_write(const float* qkv, int64_t ld, int hq, int hkv, int dk, int dv, const float* q_w, const float* k_w,
                                    float eps, float temp_coef, int temp_every, const int* positions, const int* slots,
                                    void* k_cache, void* v_cache, int block_size, void* q_out, int T_, int dtype,
                                    cudaStream_t stream) {
  LLMSS_REQUIRE(hq > 0 && hkv > 0 && temp_every > 0, "qknorm_kv_write: bad sizes");
  if (T_ <= 0) return 0;
  const int64_t units = (int64_t)T_ * (hq + 2 * hkv);
  LLMSS_BY_DTYPE(dtype, (qknorm_kv_write_kernel<T><<<(unsigned)((units + NW - 1) / NW), NW * 32, 0, stream>>>(
                            qkv, ld, hq, hkv, dk, dv, q_w, k_w, eps, temp_coef, temp_every, positions, slots, (T*)k_cache, (T*)v_cache,
                            block_size, (T*)q_out, T_)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_head_gate(void* x, int64_t ldx, const float* gate, int64_t ldg, int T_, int hq, int dv, int dtype,
                              cudaStream_t stream) {
  if (T_ <= 0) return 0;
  LLMSS_BY_DTYPE(dtype, (head_gate_kernel<T><<<T_, 256, 0, stream>>>((T*)x, ldx, gate, ldg, hq, dv)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

LLMSS_API int llmss_attention_bias(const void* q, int64_t ldq, const void* k_cache, const void* v_cache, const int* block_tables,
                                   int max_blocks, int block_size, const int* seq_lens, const int* cu_q, const float* bias,
                                   int n_dist, const float* gate, int64_t ldg, void* out, int B, int max_q, int hq, int hkv, int dk,
                                   int dv, float scale, int dtype, cudaStream_t stream) {
  LLMSS_REQUIRE(hq > 0 && hkv > 0 && hq % hkv == 0, "attention_bias: %d query heads over %d key/value heads", hq, hkv);
  LLMSS_REQUIRE(dv <= 32 * MAXV, "attention_bias: value size %d (at most %d)", dv, 32 * MAXV);
  LLMSS_REQUIRE(bias == nullptr || n_dist > 0, "attention_bias: empty bias table");
  if (B <= 0 || max_q <= 0) return 0;
  AbArgs a;
  a.q = q; a.ldq = ldq; a.k_cache = k_cache; a.v_cache = v_cache; a.block_tables = block_tables; a.max_blocks = max_blocks;
  a.bs = block_size; a.seq_lens = seq_lens; a.cu_q = cu_q; a.bias = bias; a.n_dist = n_dist; a.gate = gate; a.ldg = ldg; a.out = out;
  a.hq = hq; a.hkv = hkv; a.dk = dk; a.dv = dv; a.scale = scale;
  const int gsz = hq / hkv;
  a.nh = gsz < NW ? gsz : NW;
  a.rows = NW / a.nh;
  a.hsub = (gsz + NW - 1) / NW;
  const size_t smem = sizeof(float) * ((size_t)NW * dk + (size_t)TK * (dk + 1) + (size_t)TK * dv);
  LLMSS_REQUIRE(smem <= 200 * 1024, "attention_bias: key size %d / value size %d exceed shared memory", dk, dv);
  const dim3 grid((max_q + a.rows - 1) / a.rows, hkv * a.hsub, B);
  LLMSS_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "attention_bias: grid too large");
#define LLMSS_AB(TT)                                                                \
  do {                                                                              \
    static PerDeviceSmem gsm;                                                       \
    LLMSS_CHECK_CUDA(gsm.ensure(attention_bias_kernel<TT>, (int)smem));             \
    attention_bias_kernel<TT><<<grid, NW * 32, smem, stream>>>(a);                  \
  } while (0)
  if (dtype == LLMSS_F16) LLMSS_AB(__half);
  else if (dtype == LLMSS_BF16) LLMSS_AB(__nv_bfloat16);
  else if (dtype == LLMSS_F32) LLMSS_AB(float);
  else LLMSS_REQUIRE(false, "bad dtype %d", dtype);
#undef LLMSS_AB
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}
