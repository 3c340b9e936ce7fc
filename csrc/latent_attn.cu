// Latent (low-rank KV) attention without positional rotation, in its absorbed form, over a paged cache.
//
// A layer of this kind caches one latent vector c_j (rank R) per token instead of per-head keys and values:
//     k_{j,h} = W_uk,h c_j ,  v_{j,h} = W_uv,h c_j .
// Because no rotation sits between W_uk and the dot product, the key projection can be moved to the query
// side:  q_h . k_{j,h} = (W_uk,h^T q_h) . c_j , and the value projection behind the softmax:
//     o_h = W_uv,h ( sum_j p_{hj} c_j ).
// What remains is multi-query attention whose single shared "head" is the latent itself (K = V = c, width R),
// so every head and every query token of a sequence reads the same cache lines.
//
//   latent_prep : per token, RMS-norm the down-projected latent (32-bit) and write it to its cache slot;
//                 cast q to the compute type; output gate = sigmoid(g) per head (optional).
//   latent_attn : generic kernel, any R / head count / page size, 32-bit scores, softmax and accumulation.
//                 One CTA = one sequence x a tile of (query tokens x heads) = 16 score rows that share their
//                 key tiles; optional split of the key range (decode with few sequences) with a combine pass.
// Cache layout: [num_blocks, block_size, R] (= the [blocks, kv_heads = 1, block_size, d] layout of the
// multi-head kernels, so those can read it where R is a size they support).
#include "common.cuh"

namespace {

constexpr int ROWS = 16, TK = 32, NT = 256;

__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  return warp_sum(l < 4 ? red[l] : 0.f);
}

template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(const float* __restrict__ y, int64_t ldy, int q_off, int c_off,
                                                          int g_off, int n_q, int R, int H, const T* __restrict__ norm_w,
                                                          float eps, const int* __restrict__ slots, T* __restrict__ cache,
                                                          T* __restrict__ q_out, int64_t ldq, float* __restrict__ gate) {
  __shared__ float red[4];
  const int64_t t = blockIdx.x;
  const float* row = y + t * ldy;
  float ss = 0.f;
  for (int r = threadIdx.x; r < R; r += 128) ss += row[c_off + r] * row[c_off + r];
  ss = block_sum_128(ss, red);
  const float rstd = rsqrtf(ss / (float)R + eps);
  const int slot = slots[t];
  if (slot >= 0)
    for (int r = threadIdx.x; r < R; r += 128)
      cache[(int64_t)slot * R + r] = from_f32<T>(row[c_off + r] * rstd * to_f32(norm_w[r]));
  for (int i = threadIdx.x; i < n_q; i += 128) q_out[t * ldq + i] = from_f32<T>(row[q_off + i]);
  if (gate != nullptr)
    for (int h = threadIdx.x; h < H; h += 128) gate[t * H + h] = 1.f / (1.f + expf(-row[g_off + h]));
}

struct LaArgs {
  const float* q; int64_t ldq;       // absorbed queries [T, H * R], 32-bit
  const void* cache;                 // [slots, R]
  const int* block_tables; int max_blocks, block_size;
  const int* seq_lens; const int* cu_q;
  void* out; int64_t ldo;            // [T, H * R]
  float* part_o; float* part_ml;     // split partials: [split][T * H][R], [split][T * H][2]
  int H, R, Rp, TQ, HG, qtiles, splits, T;
  float scale;
};

// smem: Qs[ROWS][R] | Ps[ROWS][TK] | st[3][ROWS] (m, l, alpha) | slot[TK] | Cs[TK][Rp] (T)
template <typename T, typename TO, int RPT>
__global__ void __launch_bounds__(NT) latent_attn_kernel(LaArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* Qs = reinterpret_cast<float*>(smem_raw);
  float* Ps = Qs + ROWS * a.R;
  float* st_m = Ps + ROWS * TK;
  float* st_l = st_m + ROWS;
  float* st_a = st_l + ROWS;
  int* kslot = reinterpret_cast<int*>(st_a + ROWS);
  T* Cs = reinterpret_cast<T*>(kslot + TK);
  const T* cache = reinterpret_cast<const T*>(a.cache);

  const int b = blockIdx.x / a.qtiles, qt = blockIdx.x % a.qtiles;
  const int q0 = a.cu_q[b], qlen = a.cu_q[b + 1] - q0;
  const int t0 = qt * a.TQ;
  if (t0 >= qlen) return;
  const int h0 = blockIdx.y * a.HG;
  const int ctx = a.seq_lens[b] - qlen;              // tokens cached before this step's
  const int nt = min(a.TQ, qlen - t0);               // query tokens of this tile
  const int kend = ctx + t0 + nt;                    // keys [0, kend) are visible to the tile's last token
  const int ntiles = (kend + TK - 1) / TK;
  const int per = (ntiles + a.splits - 1) / a.splits;
  const int tile_lo = blockIdx.z * per, tile_hi = min(ntiles, tile_lo + per);
  const int R = a.R, Rp = a.Rp, HG = a.HG;
  const int nrows = nt * HG;                         // row r: token t0 + r / HG, head h0 + r % HG

  for (int idx = threadIdx.x; idx < ROWS * R; idx += NT) {
    const int r = idx / R, c = idx % R;
    const int h = h0 + r % HG;
    float v = 0.f;
    if (r < nrows && h < a.H) v = a.q[(int64_t)(q0 + t0 + r / HG) * a.ldq + (int64_t)h * R + c] * a.scale;
    Qs[idx] = v;
  }
  if (threadIdx.x < ROWS) { st_m[threadIdx.x] = -INFINITY; st_l[threadIdx.x] = 0.f; }
  float acc[ROWS][RPT];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int c = 0; c < RPT; ++c) acc[r][c] = 0.f;
  __syncthreads();

  const int* bt = a.block_tables + (int64_t)b * a.max_blocks;
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int j0 = tile * TK;
    if (threadIdx.x < TK) {
      const int kj = j0 + threadIdx.x;
      kslot[threadIdx.x] = kj < kend ? bt[kj / a.block_size] * a.block_size + kj % a.block_size : -1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < TK * R; idx += NT) {
      const int j = idx / R, c = idx % R;
      const int s = kslot[j];
      Cs[j * Rp + c] = s >= 0 ? cache[(int64_t)s * R + c] : from_f32<T>(0.f);
    }
    __syncthreads();
    // scores: lane = key, warp w takes rows w and w + 8
    {
      const int j = threadIdx.x & 31;
      const T* cj = Cs + j * Rp;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int r = (threadIdx.x >> 5) + rr * 8;
        const float* qr = Qs + r * R;
        float s = 0.f;
        for (int c = 0; c < R; ++c) s = fmaf(qr[c], to_f32(cj[c]), s);
        const int pos = ctx + t0 + r / HG;           // absolute position of the row's query
        const bool ok = r < nrows && (j0 + j) <= pos;
        s = ok ? s : -INFINITY;
        // online softmax of the row across the warp
        const float mx = warp_max(s);
        const float m_old = st_m[r];
        const float m_new = fmaxf(m_old, mx);
        const float p = (m_new == -INFINITY) ? 0.f : expf(s - m_new);
        const float sum = warp_sum(p);
        Ps[r * TK + j] = p;
        __syncwarp();
        if (j == 0) {
          const float al = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
          st_a[r] = al;
          st_l[r] = st_l[r] * al + sum;
          st_m[r] = m_new;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float al = st_a[r];
#pragma unroll
      for (int c = 0; c < RPT; ++c) acc[r][c] *= al;
    }
    for (int j = 0; j < TK; ++j) {
      float cv[RPT];
#pragma unroll
      for (int c = 0; c < RPT; ++c) {
        const int col = threadIdx.x + c * NT;
        cv[c] = col < R ? to_f32(Cs[j * Rp + col]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const float p = Ps[r * TK + j];
#pragma unroll
        for (int c = 0; c < RPT; ++c) acc[r][c] = fmaf(p, cv[c], acc[r][c]);
      }
    }
    __syncthreads();
  }

  // epilogue
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int h = h0 + r % HG;
    if (r >= nrows || h >= a.H) continue;
    const int64_t trow = q0 + t0 + r / HG;
    if (a.splits == 1) {
      const float l = st_l[r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      TO* o = reinterpret_cast<TO*>(a.out) + trow * a.ldo + (int64_t)h * R;
#pragma unroll
      for (int c = 0; c < RPT; ++c) {
        const int col = threadIdx.x + c * NT;
        if (col < R) o[col] = from_f32<TO>(acc[r][c] * inv);
      }
    } else {
      const int64_t pr = ((int64_t)blockIdx.z * a.T + trow) * a.H + h;
      float* o = a.part_o + pr * R;
#pragma unroll
      for (int c = 0; c < RPT; ++c) {
        const int col = threadIdx.x + c * NT;
        if (col < R) o[col] = acc[r][c];
      }
      if (threadIdx.x == 0) { a.part_ml[pr * 2] = st_m[r]; a.part_ml[pr * 2 + 1] = st_l[r]; }
    }
  }
}

template <typename TO>
__global__ void __launch_bounds__(128) latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                             TO* __restrict__ out, int64_t ldo, int T, int H, int R, int splits) {
  const int64_t th = blockIdx.x;                   // token * H + head
  const int64_t t = th / H, h = th % H;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[((int64_t)s * T * H + th) * 2]);
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = part_ml[((int64_t)s * T * H + th) * 2], l = part_ml[((int64_t)s * T * H + th) * 2 + 1];
    if (m != -INFINITY) L += l * expf(m - M);
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int c = threadIdx.x; c < R; c += 128) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = part_ml[((int64_t)s * T * H + th) * 2];
      if (m != -INFINITY) v += part_o[((int64_t)s * T * H + th) * R + c] * expf(m - M);
    }
    out[t * ldo + h * R + c] = from_f32<TO>(v * inv);
  }
}

template <typename T, typename TO>
int launch_la(const LaArgs& a, int num_seqs, cudaStream_t stream) {
  const int rpt = (a.R + NT - 1) / NT;
  const size_t smem = (size_t)(ROWS * a.R + ROWS * TK + 3 * ROWS) * 4 + TK * 4 + (size_t)TK * a.Rp * sizeof(T);
  dim3 grid(num_seqs * a.qtiles, (a.H + a.HG - 1) / a.HG, a.splits);
#define LLMSS_LA(RPT_)                                                                                   \
  {                                                                                                      \
    static PerDeviceSmem granted;                                                                        \
    LLMSS_CHECK_CUDA(granted.ensure(latent_attn_kernel<T, TO, RPT_>, (int)smem));                        \
    latent_attn_kernel<T, TO, RPT_><<<grid, NT, smem, stream>>>(a);                                      \
  }
  if (rpt <= 1) LLMSS_LA(1)
  else if (rpt <= 2) LLMSS_LA(2)
  else LLMSS_LA(4)
#undef LLMSS_LA
  LLMSS_CHECK_CUDA(cudaGetLastError());
  if (a.splits > 1) {
    latent_combine_kernel<TO><<<a.T * a.H, 128, 0, stream>>>(a.part_o, a.part_ml, reinterpret_cast<TO*>(a.out), a.ldo, a.T,
                                                             a.H, a.R, a.splits);
    LLMSS_CHECK_CUDA(cudaGetLastError());
  }
  return 0;
}

}  // namespace

LLMSS_API int llmss_latent_prep(const float* y, int64_t ldy, int q_off, int c_off, int g_off, int n_q, int R, int H,
                                const void* norm_w, float eps, const int* slots, void* cache, void* q_out, int64_t ldq,
                                float* gate, int T_, int dtype, cudaStream_t stream) {
  if (T_ == 0) return 0;
  LLMSS_BY_DTYPE(dtype, (latent_prep_kernel<T><<<T_, 128, 0, stream>>>(y, ldy, q_off, c_off, g_off, n_q, R, H, (const T*)norm_w,
                                                                      eps, slots, (T*)cache, (T*)q_out, ldq, gate)));
  LLMSS_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// floats of scratch the split form needs (partials + their (max, sum) pairs)
LLMSS_API int64_t llmss_latent_attn_scratch_floats(int T_, int H, int R, int splits) {
  return splits > 1 ? (int64_t)splits * T_ * H * (R + 2) : 0;
}

// out_f32: the context is written in 32-bit (true 32-bit mode), else in the cache's type.
LLMSS_API int llmss_latent_attn(const float* q, int64_t ldq, const void* cache, const int* block_tables, int max_blocks,
                                int block_size, const int* seq_lens, const int* cu_q, void* out, int64_t ldo, float* scratch,
                                int T_, int num_seqs, int max_q, int H, int R, float scale, int splits, int dtype,
                                cudaStream_t stream) {
  LLMSS_REQUIRE(H > 0 && R > 0 && R <= 4 * NT, "latent_attn: rank %d not in 1..%d", R, 4 * NT);
  LLMSS_REQUIRE(splits >= 1 && (splits == 1 || scratch != nullptr), "latent_attn: split form needs scratch");
  if (T_ == 0 || num_seqs == 0) return 0;
  LaArgs a;
  a.q = q; a.ldq = ldq; a.cache = cache; a.block_tables = block_tables; a.max_blocks = max_blocks; a.block_size = block_size;
  a.seq_lens = seq_lens; a.cu_q = cu_q; a.out = out; a.ldo = ldo;
  a.H = H; a.R = R; a.T = T_; a.scale = scale; a.splits = splits;
  a.HG = H < ROWS ? H : ROWS;
  a.TQ = max_q <= 1 ? 1 : ROWS / a.HG;
  a.qtiles = (max_q + a.TQ - 1) / a.TQ;
  a.part_o = scratch;
  a.part_ml = scratch != nullptr ? scratch + (int64_t)splits * T_ * H * R : nullptr;
  // row stride of the key tile in shared memory: an odd number of 32-bit words, so that the 32 keys a warp
  // reads in the score loop fall into 32 different banks
  const int esz = dtype == LLMSS_F32 ? 4 : 2;
  int Rp = R;
  if (esz == 4) { if (Rp % 2 == 0) Rp += 1; }
  else { Rp += Rp % 2; if ((Rp / 2) % 2 == 0) Rp += 2; }
  a.Rp = Rp;
  const size_t smem = (size_t)(ROWS * R + ROWS * TK + 3 * ROWS) * 4 + TK * 4 + (size_t)TK * Rp * esz;
  LLMSS_REQUIRE(smem <= 227 * 1024, "latent_attn: rank %d needs %zu bytes of shared memory", R, smem);
  if (dtype == LLMSS_F32) return launch_la<float, float>(a, num_seqs, stream);
  if (dtype == LLMSS_BF16) return launch_la<__nv_bfloat16, __nv_bfloat16>(a, num_seqs, stream);
  if (dtype == LLMSS_F16) return launch_la<__half, __half>(a, num_seqs, stream);
  LLMSS_REQUIRE(false, "latent_attn: bad dtype %d", dtype);
}
