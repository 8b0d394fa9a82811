// Softmax attention whose scores are mixed across the heads before the softmax ("talking heads"):
//     s_g(i, j) = scale * q_g(i) . k_kv(g)(j)                for every query head g
//     t_h(i, j) = sum_g talk[h, g] * s_g(i, j)               mixed with a learned [H, H] matrix
//     p_h(i, :) = softmax over the visible j of t_h(i, :)    j <= i, and i - j < window when there is a window
//     o_h(i)    = sum_j p_h(i, j) * v_kv(h)(j)               (then times sigmoid(gate) where a gate is given)
// over the paged cache (keys [page][kv head][position][dim], values [page][kv head][dim][position]).
//
// A head's weights depend on every head's scores, so a block takes ALL heads of a few query rows of one
// sequence and walks the key range in tiles: the tile's keys and values of every kv head go to shared memory,
// each warp forms the raw scores of its (row, head) pairs with a lane per key, the pairs' scores meet in
// shared memory, each warp mixes, masks and runs the streaming softmax for its pairs (lane = key), and adds
// the weighted values with a lane per value dimension.  Scores, mixing, softmax and sums are float whatever
// the cache holds.  The same kernel serves prompts, portions and decode steps; a decode step may cut the key
// range over several blocks (partial maximum, sum and values to scratch, merged by a second kernel).
#include "common.cuh"

#define AMX_NEG (-1e30f)
constexpr int AMX_MAX_WARPS = 16;

template <typename T> struct AmxPiece;      // a 16-byte piece of a cached row as floats
template <> struct AmxPiece<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
};
template <> struct AmxPiece<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const bf16* p, float* f) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// Shared memory, in this order: talk [H*H] | q [NP][hdp] | raw [NP][KT] | p [NP][KT] (floats), then
// keys [G][KT][KS] and values [G][KT][vdp] in the cache's type.  NP = QT * H pairs; pair = row * H + head.
template <typename T, int HDL, int RPW>
__global__ void __launch_bounds__(32 * AMX_MAX_WARPS)
attention_mixed_kernel(T* __restrict__ out, float* __restrict__ part, const T* __restrict__ q, int ldq,
                       const T* __restrict__ k_pool, const T* __restrict__ v_pool, const int* __restrict__ block_table,
                       int bt_width, const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0,
                       const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen, const float* __restrict__ talk,
                       const float* __restrict__ gate, int ldg, int H, int G, int hd, int vd, int page_size, int window,
                       float scale, int QT, int KT, int n_splits) {
  extern __shared__ __align__(16) unsigned char amx_sm[];
  constexpr int EV = AmxPiece<T>::N;
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int b = blockIdx.z, split = blockIdx.y;
  const int slot = seq_slot[b];
  const int qlen = seq_qlen ? seq_qlen[b] : 1;
  const int row_lo = blockIdx.x * QT;
  if (row_lo >= qlen) return;
  const int nrows = min(QT, qlen - row_lo);
  const int q0 = seq_qstart[b], pos0 = seq_pos0[b];
  const int Gq = H / G;
  const int NP = QT * H;
  const int hdp = (hd + 7) & ~7, KS = hdp + EV, vdp = (vd + 7) & ~7;

  float* talk_s = reinterpret_cast<float*>(amx_sm);
  float* q_s = talk_s + ((H * H + 3) & ~3);
  float* raw_s = q_s + (size_t)NP * hdp;
  float* p_s = raw_s + (size_t)NP * KT;
  T* k_s = reinterpret_cast<T*>(p_s + (size_t)NP * KT);
  T* v_s = k_s + (size_t)G * KT * KS;

  // this warp's pairs: warp + nw * r
  int pr_i[RPW], pr_h[RPW], pr_c[RPW];
  bool pr_on[RPW];
  bool same_c = true;
#pragma unroll
  for (int r = 0; r < RPW; r++) {
    const int p = warp + nw * r;
    pr_i[r] = p / H;
    pr_h[r] = p - pr_i[r] * H;
    pr_c[r] = pr_h[r] / Gq;
    pr_on[r] = p < NP && pr_i[r] < nrows;
    if (p >= NP) { pr_i[r] = 0; pr_h[r] = 0; pr_c[r] = 0; }
    if (pr_c[r] != pr_c[0]) same_c = false;
  }

  if (slot < 0) {      // a padding sequence: a defined result, no cache access
#pragma unroll
    for (int r = 0; r < RPW; r++) {
      if (!pr_on[r]) continue;
      const size_t m = (size_t)q0 + row_lo + pr_i[r];
      if (n_splits == 1) {
        for (int d = lane; d < vd; d += 32) out[(m * H + pr_h[r]) * vd + d] = from_f32<T>(0.f);
      } else {
        float* pp = part + ((m * H + pr_h[r]) * n_splits + split) * (size_t)(vd + 2);
        if (lane == 0) { pp[0] = AMX_NEG; pp[1] = 0.f; }
        for (int d = lane; d < vd; d += 32) pp[2 + d] = 0.f;
      }
    }
    return;
  }

  for (int idx = threadIdx.x; idx < H * H; idx += blockDim.x) talk_s[idx] = talk[idx];
  for (int idx = threadIdx.x; idx < NP * hdp; idx += blockDim.x) {
    const int p = idx / hdp, d = idx - p * hdp;
    const int i = p / H, h = p - i * H;
    float v = 0.f;
    if (i < nrows && d < hd) v = to_f32(q[(size_t)(q0 + row_lo + i) * ldq + (size_t)h * hd + d]);
    q_s[idx] = v;
  }

  const int kv_len = pos0 + qlen;
  const int pos_lo = pos0 + row_lo, pos_hi = pos_lo + nrows - 1;
  const int key_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
  const int tile_first = key_lo / KT, n_tiles = pos_hi / KT - tile_first + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int t_lo = split * per_split, t_hi = min(n_tiles, t_lo + per_split);

  float mx[RPW], l[RPW], acc[RPW][HDL];
#pragma unroll
  for (int r = 0; r < RPW; r++) {
    mx[r] = AMX_NEG;
    l[r] = 0.f;
#pragma unroll
    for (int jj = 0; jj < HDL; jj++) acc[r][jj] = 0.f;
  }
  const bool kvec = hd % EV == 0;
  const int jc = lane < KT ? lane : KT - 1;      // lanes beyond the tile's keys compute on its last key and are ignored

  for (int ut = t_lo; ut < t_hi; ut++) {
    const int key0 = (tile_first + ut) * KT;
    const int page = block_table[(size_t)b * bt_width + key0 / page_size];
    const int in_page = key0 % page_size;
    __syncthreads();      // the tile before is used up (and q, talk are in place)
    // keys: [c][j][0..hdp) with zeros behind hd and for positions that hold nothing yet
    if (kvec) {
      const int per_row = hdp / EV, total = G * KT * per_row;
      for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int c = idx / (KT * per_row), rest = idx - c * (KT * per_row);
        const int j = rest / per_row, d0 = (rest - j * per_row) * EV;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (page >= 0 && key0 + j < kv_len && d0 < hd)
          v = *reinterpret_cast<const uint4*>(k_pool + (((size_t)page * G + c) * page_size + in_page + j) * hd + d0);
        *reinterpret_cast<uint4*>(k_s + ((size_t)c * KT + j) * KS + d0) = v;
      }
    } else {
      const int total = G * KT * hdp;
      for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int c = idx / (KT * hdp), rest = idx - c * (KT * hdp);
        const int j = rest / hdp, d = rest - j * hdp;
        T v = from_f32<T>(0.f);
        if (page >= 0 && key0 + j < kv_len && d < hd)
          v = k_pool[(((size_t)page * G + c) * page_size + in_page + j) * hd + d];
        k_s[((size_t)c * KT + j) * KS + d] = v;
      }
    }
    // values: cached [dim][position], staged [c][j][dim]; a thread takes EV positions of one dimension, and the
    // threads of a warp neighbouring dimensions (their stores fall in different banks)
    {
      const int chunks = KT / EV, total = G * chunks * vd;
      for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const int c = idx / (chunks * vd), rest = idx - c * (chunks * vd);
        const int ch = rest / vd, d = rest - ch * vd;
        float f[EV];
#pragma unroll
        for (int u = 0; u < EV; u++) f[u] = 0.f;
        if (page >= 0)
          AmxPiece<T>::load(v_pool + (((size_t)page * G + c) * vd + d) * page_size + in_page + ch * EV, f);
#pragma unroll
        for (int u = 0; u < EV; u++) {
          const int j = ch * EV + u;
          v_s[((size_t)c * KT + j) * vdp + d] = from_f32<T>(key0 + j < kv_len ? f[u] : 0.f);
        }
      }
    }
    __syncthreads();
    // raw scores of this warp's pairs, a lane per key
    {
      float sc[RPW];
#pragma unroll
      for (int r = 0; r < RPW; r++) sc[r] = 0.f;
      if (same_c) {
        const T* kr = k_s + ((size_t)pr_c[0] * KT + jc) * KS;
        for (int d0 = 0; d0 < hdp; d0 += EV) {
          float kf[EV];
          AmxPiece<T>::load(kr + d0, kf);
#pragma unroll
          for (int r = 0; r < RPW; r++) {
            const float* qr = q_s + (size_t)(warp + nw * r < NP ? warp + nw * r : 0) * hdp + d0;
#pragma unroll
            for (int u = 0; u < EV; u += 4) {
              const float4 qv = *reinterpret_cast<const float4*>(qr + u);
              sc[r] = fmaf(qv.x, kf[u], sc[r]);
              sc[r] = fmaf(qv.y, kf[u + 1], sc[r]);
              sc[r] = fmaf(qv.z, kf[u + 2], sc[r]);
              sc[r] = fmaf(qv.w, kf[u + 3], sc[r]);
            }
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < RPW; r++) {
          const T* kr = k_s + ((size_t)pr_c[r] * KT + jc) * KS;
          const float* qr = q_s + (size_t)(warp + nw * r < NP ? warp + nw * r : 0) * hdp;
          for (int d0 = 0; d0 < hdp; d0 += EV) {
            float kf[EV];
            AmxPiece<T>::load(kr + d0, kf);
#pragma unroll
            for (int u = 0; u < EV; u += 4) {
              const float4 qv = *reinterpret_cast<const float4*>(qr + d0 + u);
              sc[r] = fmaf(qv.x, kf[u], sc[r]);
              sc[r] = fmaf(qv.y, kf[u + 1], sc[r]);
              sc[r] = fmaf(qv.z, kf[u + 2], sc[r]);
              sc[r] = fmaf(qv.w, kf[u + 3], sc[r]);
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RPW; r++)
        if (warp + nw * r < NP && lane < KT) raw_s[(size_t)(warp + nw * r) * KT + lane] = sc[r] * scale;
    }
    __syncthreads();
    // mixing across heads, mask, streaming softmax; the weights of the tile to p_s
#pragma unroll
    for (int r = 0; r < RPW; r++) {
      if (warp + nw * r >= NP) continue;      // warp-uniform
      const int p = warp + nw * r;
      const int pos = pos_lo + pr_i[r], key = key0 + lane;
      float t = 0.f;
      if (lane < KT) {
        const float* row = raw_s + (size_t)pr_i[r] * H * KT + lane;
        const float* tk = talk_s + pr_h[r] * H;
        for (int g = 0; g < H; g++) t = fmaf(tk[g], row[(size_t)g * KT], t);
      }
      const bool seen = lane < KT && pr_on[r] && key <= pos && (window <= 0 || pos - key < window);
      const float tmax = warp_max(seen ? t : AMX_NEG);
      const float m_new = fmaxf(mx[r], tmax);
      const float w = seen ? expf(t - m_new) : 0.f;
      const float corr = expf(mx[r] - m_new);      // 1 while nothing was seen (both at the floor)
      l[r] = l[r] * corr + warp_sum(w);
      mx[r] = m_new;
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) acc[r][jj] *= corr;
      if (lane < KT) p_s[(size_t)p * KT + lane] = w;
    }
    __syncwarp();
    // weighted values, a lane per dimension; four keys' weights per read
    if (same_c) {
      const T* vb = v_s + (size_t)pr_c[0] * KT * vdp;
      for (int j = 0; j < KT; j += 4) {
        float4 pw[RPW];
#pragma unroll
        for (int r = 0; r < RPW; r++)
          pw[r] = *reinterpret_cast<const float4*>(p_s + (size_t)(warp + nw * r < NP ? warp + nw * r : 0) * KT + j);
#pragma unroll
        for (int jj = 0; jj < HDL; jj++) {
          const int d = lane + 32 * jj;
          if (d >= vd) break;
          const float v0 = to_f32(vb[(size_t)(j + 0) * vdp + d]), v1 = to_f32(vb[(size_t)(j + 1) * vdp + d]);
          const float v2 = to_f32(vb[(size_t)(j + 2) * vdp + d]), v3 = to_f32(vb[(size_t)(j + 3) * vdp + d]);
#pragma unroll
          for (int r = 0; r < RPW; r++) {
            acc[r][jj] = fmaf(pw[r].x, v0, acc[r][jj]);
            acc[r][jj] = fmaf(pw[r].y, v1, acc[r][jj]);
            acc[r][jj] = fmaf(pw[r].z, v2, acc[r][jj]);
            acc[r][jj] = fmaf(pw[r].w, v3, acc[r][jj]);
          }
        }
      }
    } else {
#pragma unroll
      for (int r = 0; r < RPW; r++) {
        if (warp + nw * r >= NP) continue;
        const T* vb = v_s + (size_t)pr_c[r] * KT * vdp;
        const float* pw = p_s + (size_t)(warp + nw * r) * KT;
        for (int j = 0; j < KT; j += 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(pw + j);
#pragma unroll
          for (int jj = 0; jj < HDL; jj++) {
            const int d = lane + 32 * jj;
            if (d >= vd) break;
            acc[r][jj] = fmaf(w4.x, to_f32(vb[(size_t)(j + 0) * vdp + d]), acc[r][jj]);
            acc[r][jj] = fmaf(w4.y, to_f32(vb[(size_t)(j + 1) * vdp + d]), acc[r][jj]);
            acc[r][jj] = fmaf(w4.z, to_f32(vb[(size_t)(j + 2) * vdp + d]), acc[r][jj]);
            acc[r][jj] = fmaf(w4.w, to_f32(vb[(size_t)(j + 3) * vdp + d]), acc[r][jj]);
          }
        }
      }
    }
  }

#pragma unroll
  for (int r = 0; r < RPW; r++) {
    if (!pr_on[r]) continue;
    const size_t m = (size_t)q0 + row_lo + pr_i[r];
    const int h = pr_h[r];
    if (n_splits == 1) {
      const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d >= vd) break;
        float o = acc[r][jj] * inv;
        if (gate) o *= 1.0f / (1.0f + expf(-gate[m * ldg + (size_t)h * vd + d]));
        out[(m * H + h) * vd + d] = from_f32<T>(o);
      }
    } else {
      float* pp = part + ((m * H + h) * n_splits + split) * (size_t)(vd + 2);
      if (lane == 0) { pp[0] = mx[r]; pp[1] = l[r]; }
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < vd) pp[2 + d] = acc[r][jj];
      }
    }
  }
}

// The pieces of a cut key range put together: a warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(128)
attention_mixed_merge_kernel(T* __restrict__ out, const float* __restrict__ part, const float* __restrict__ gate, int ldg,
                             size_t pairs, int H, int vd, int n_splits) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t pair = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const float* pp = part + pair * n_splits * (size_t)(vd + 2);
  float m = AMX_NEG;
  for (int s = 0; s < n_splits; s++) m = fmaxf(m, pp[(size_t)s * (vd + 2)]);
  float l = 0.f;
  for (int s = 0; s < n_splits; s++) l += pp[(size_t)s * (vd + 2) + 1] * expf(pp[(size_t)s * (vd + 2)] - m);
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  const size_t row = pair / H;
  const int h = (int)(pair - row * H);
  for (int d = lane; d < vd; d += 32) {
    float a = 0.f;
    for (int s = 0; s < n_splits; s++) a += pp[(size_t)s * (vd + 2) + 2 + d] * expf(pp[(size_t)s * (vd + 2)] - m);
    float o = a * inv;
    if (gate) o *= 1.0f / (1.0f + expf(-gate[row * ldg + (size_t)h * vd + d]));
    out[pair * vd + d] = from_f32<T>(o);
  }
}

// ---- prompts in bfloat16 on the tensor cores ---------------------------------------------------------------
// The same attention for the many rows of a prompt.  A block of 16 warps takes 16 query rows of one sequence and
// ALL heads, and walks the key range in tiles of 32 keys:
//   1. the tile's keys of every kv head go to shared memory; every warp forms raw score tiles S_g = Q_g K^T
//      (16 rows x 8 keys, mma.sync m16n8k16, bfloat16 operands, float sums) for its share of the (head, 8 keys)
//      pairs and leaves them, times the scale, in shared memory as floats;
//   2. warp i takes row i, first with a lane per key: it reads the row's raw scores of all heads once, mixes them
//      into every head's score with the [heads, heads] matrix (float multiply-adds, the matrix transposed in
//      shared memory so that four heads' factors are one load), masks, and puts the mixed scores back over the raw
//      ones; then with a lane per head: lane h reads head h's 32 scores of the row (16 bytes a load), and runs the
//      streaming softmax on them in its own registers (no exchange between lanes; lane h keeps head h's running
//      maximum and sum); the weights go back over the scores as two bfloat16 terms, hi = bf16(p) and
//      lo = bf16(p - hi), so that the product with the values sees 16 significant bits of p; meanwhile the
//      tile's values arrive in the buffer the keys have left;
//   3. every warp adds P V for its share of the (head, 8 value dimensions) pairs (two products, hi and lo),
//      after scaling its sums by the factor the softmax left for (head, row).
// Float everywhere outside the products' operands.  Sizes: up to 32 heads, key heads in multiples of 16 numbers,
// value heads in multiples of 8, heads x value size up to 2,048 (a thread then holds 64 sums).
constexpr int AMM_ROWS = 16, AMM_KT = 32, AMM_WARPS = 16, AMM_SLOT = 36, AMM_ROW_PAD = 4;

__device__ __forceinline__ void amm_mma(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four 8 x 8 tiles of 16-bit numbers from shared memory, a row (16 bytes) per lane's address: the A operand of a product.
__device__ __forceinline__ void amm_ldsm4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
// Two tiles: the B operand (lanes 0..15 give the addresses).
__device__ __forceinline__ void amm_ldsm2(uint32_t& r0, uint32_t& r1, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
               : "=r"(r0), "=r"(r1) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
// Two float multiply-adds in one instruction (sm_100): acc = a * b + acc on both halves of the 64-bit registers.
__device__ __forceinline__ void amm_fma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long amm_pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void amm_unpack2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ float amm_exp2(float x) {      // 2^x from the special function unit (relative error about 2^-22)
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Shared memory: talkT [H][HP] floats | corr [H][16] floats | raw / P [16][H][AMM_SLOT] (+ AMM_ROW_PAD a row) floats
// (a (row, head)'s 32 raw scores, then its mixed scores, then its weights: hi in the first 16 words, lo in the
// next 16; the strides keep the products' fragment loads, a lane per key and a lane per head all off each other's
// banks) | q [H][16][hd + 8] bfloat16 | keys [G][32][hd + 8] or values [G][vd][40] bfloat16 (one buffer).
template <int HP, int UPW, bool AHEAD>
__global__ void __launch_bounds__(32 * AMM_WARPS, 1)
attention_mixed_mma_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, int ldq, const bf16* __restrict__ k_pool,
                           const bf16* __restrict__ v_pool, const int* __restrict__ block_table, int bt_width,
                           const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0,
                           const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                           const float* __restrict__ talk, const float* __restrict__ gate, int ldg, int H, int G, int hd,
                           int vd, int page_size, int window, float scale) {
  extern __shared__ __align__(16) unsigned char amm_sm[];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gid = lane >> 2, tig = lane & 3;
  const int b = blockIdx.y;
  const int slot = seq_slot[b];
  const int qlen = seq_qlen ? seq_qlen[b] : 1;
  const int row_lo = blockIdx.x * AMM_ROWS;
  if (row_lo >= qlen) return;
  const int nrows = min(AMM_ROWS, qlen - row_lo);
  const int q0 = seq_qstart[b], pos0 = seq_pos0[b];
  const int Gq = H / G;
  const int QS = hd + 8, KS = hd + 8, VS = AMM_KT + 8;
  const int n_dt = vd / 8;                       // tiles of 8 value dimensions in a head
  const int n_units = H * n_dt;                  // (head, dimension tile) pairs of the block

  float* talkT = reinterpret_cast<float*>(amm_sm);            // [g][HP]
  float* corr_s = talkT + H * HP;                             // [h][16]
  float* raw_s = corr_s + H * AMM_ROWS;                       // [h][16][AMM_SLOT]
  const int RS = H * AMM_SLOT + AMM_ROW_PAD;                  // words of a row of raw_s
  bf16* q_s = reinterpret_cast<bf16*>(raw_s + (size_t)AMM_ROWS * RS);   // [g][16][QS]
  bf16* kv_s = q_s + (size_t)H * AMM_ROWS * QS;

  if (slot < 0) {      // a padding sequence: a defined result, no cache access
    for (int idx = threadIdx.x; idx < nrows * H * vd; idx += blockDim.x)
      out[(size_t)(q0 + row_lo) * H * vd + idx] = __float2bfloat16_rn(0.f);
    return;
  }
  for (int idx = threadIdx.x; idx < H * HP; idx += blockDim.x) {
    const int g = idx / HP, h = idx - g * HP;
    talkT[idx] = h < H ? talk[h * H + g] : 0.f;
  }
  {      // queries: [g][i][hd] with zero rows beyond the block's rows, 16 bytes at a time
    const int per_row = hd / 8, total = H * AMM_ROWS * per_row;
    for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
      const int g = idx / (AMM_ROWS * per_row), rest = idx - g * (AMM_ROWS * per_row);
      const int i = rest / per_row, d0 = (rest - i * per_row) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (i < nrows) v = *reinterpret_cast<const uint4*>(q + (size_t)(q0 + row_lo + i) * ldq + (size_t)g * hd + d0);
      *reinterpret_cast<uint4*>(q_s + ((size_t)g * AMM_ROWS + i) * QS + d0) = v;
    }
  }
  const int kv_len = pos0 + qlen;
  const int pos_lo = pos0 + row_lo, pos_hi = pos_lo + nrows - 1;
  const int key_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
  const int tile_first = key_lo / AMM_KT, n_tiles = pos_hi / AMM_KT - tile_first + 1;

  float acc[UPW][4];
#pragma unroll
  for (int u = 0; u < UPW; u++)
#pragma unroll
    for (int x = 0; x < 4; x++) acc[u][x] = 0.f;
  // AHEAD: a thread holds up to four 16-byte pieces of the next tile's keys while this tile's values are multiplied
  // (the launch asks for it where the sums leave the registers for it)
  constexpr int KPT = AHEAD ? 4 : 1;
  uint4 kreg[KPT];
  const int k_per_row = hd / 8, k_total = G * AMM_KT * k_per_row;
  const bool k_ahead = AHEAD;
  float m_run = AMX_NEG, l_run = 0.f;      // of head `lane` and row `warp`, kept by that lane alone
  const float scale2 = scale * 1.4426950408889634f;

  for (int ut = 0; ut < n_tiles; ut++) {
    const int key0 = (tile_first + ut) * AMM_KT;
    const int page = block_table[(size_t)b * bt_width + key0 / page_size];
    const int in_page = key0 % page_size;
    __syncthreads();      // the buffer is free (the values of the tile before are used up); q and talkT are in place
    if (k_ahead && ut > 0) {      // the keys were asked for while the tile before multiplied its values
#pragma unroll
      for (int x = 0; x < KPT; x++) {
        const int idx = threadIdx.x + x * blockDim.x;
        if (idx < k_total) {
          const int cj = idx / k_per_row, d0 = (idx - cj * k_per_row) * 8;
          *reinterpret_cast<uint4*>(kv_s + (size_t)cj * KS + d0) = kreg[x];
        }
      }
    } else {      // keys [c][j][hd]
      for (int idx = threadIdx.x; idx < k_total; idx += blockDim.x) {
        const int cj = idx / k_per_row, d0 = (idx - cj * k_per_row) * 8;
        const int c = cj / AMM_KT, j = cj - c * AMM_KT;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (page >= 0 && key0 + j < kv_len)
          v = *reinterpret_cast<const uint4*>(k_pool + (((size_t)page * G + c) * page_size + in_page + j) * hd + d0);
        *reinterpret_cast<uint4*>(kv_s + (size_t)cj * KS + d0) = v;
      }
    }
    __syncthreads();
    // 1. raw scores, a head a unit: the head's query fragments stay in registers over the tile's four groups of 8 keys.
    //    The scale carries log2(e), so the softmax below works with powers of two.
    for (int g = warp; g < H; g += AMM_WARPS) {
      const bf16* qa = q_s + (size_t)g * AMM_ROWS * QS + (size_t)(lane & 15) * QS + 8 * (lane >> 4);
      const bf16* kb = kv_s + ((size_t)(g / Gq) * AMM_KT + (lane & 7)) * KS + 8 * ((lane >> 3) & 1);
      float d[AMM_KT / 8][4];
#pragma unroll
      for (int nt = 0; nt < AMM_KT / 8; nt++) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
      for (int k0 = 0; k0 < hd; k0 += 16) {
        uint32_t a[4];
        amm_ldsm4(a, qa + k0);
#pragma unroll
        for (int nt = 0; nt < AMM_KT / 8; nt++) {
          uint32_t b0, b1;
          amm_ldsm2(b0, b1, kb + (size_t)nt * 8 * KS + k0);
          amm_mma(d[nt], a, b0, b1);
        }
      }
#pragma unroll
      for (int nt = 0; nt < AMM_KT / 8; nt++) {
        float* r0 = raw_s + (size_t)gid * RS + g * AMM_SLOT + nt * 8 + 2 * tig;
        float* r1 = raw_s + (size_t)(gid + 8) * RS + g * AMM_SLOT + nt * 8 + 2 * tig;
        *reinterpret_cast<float2*>(r0) = make_float2(d[nt][0] * scale2, d[nt][1] * scale2);
        *reinterpret_cast<float2*>(r1) = make_float2(d[nt][2] * scale2, d[nt][3] * scale2);
      }
    }
    __syncthreads();      // the scores are complete; the keys are used up
    // the tile's values on their way: asked for now, stored after the softmax
    constexpr int VPT = 4;      // 16-byte pieces of the values a thread takes (G * vd * 4 pieces in all)
    uint4 vreg[VPT];
    const int v_total = G * vd * (AMM_KT / 8);
#pragma unroll
    for (int x = 0; x < VPT; x++) {
      const int idx = threadIdx.x + x * blockDim.x;
      vreg[x] = make_uint4(0, 0, 0, 0);
      if (idx < v_total && page >= 0) {
        const int cd = idx / (AMM_KT / 8), ch = idx - cd * (AMM_KT / 8);      // cd = c * vd + d
        vreg[x] = *reinterpret_cast<const uint4*>(v_pool + ((size_t)page * G * vd + cd) * page_size + in_page + ch * 8);
      }
    }
    // 2. row `warp`: mix the heads' scores, mask, streaming softmax of every head, weights as two bfloat16 terms
    {
      const int i = warp;
      const int pos = pos_lo + i, key = key0 + lane;
      const bool seen = i < nrows && key <= pos && (window <= 0 || pos - key < window);
      unsigned long long t2[HP / 2];      // two heads' sums a register pair
#pragma unroll
      for (int h = 0; h < HP / 2; h++) t2[h] = 0ull;
      float* row = raw_s + (size_t)i * RS;
#pragma unroll 4
      for (int g = 0; g < H; g++) {
        const float r = row[g * AMM_SLOT + lane];
        const unsigned long long rr = amm_pack2(r, r);
        const ulonglong2* tk = reinterpret_cast<const ulonglong2*>(talkT + g * HP);
#pragma unroll
        for (int h4 = 0; h4 < HP / 4; h4++) {
          const ulonglong2 w4 = tk[h4];
          amm_fma2(t2[2 * h4], w4.x, rr);
          amm_fma2(t2[2 * h4 + 1], w4.y, rr);
        }
      }
      float t[HP];
#pragma unroll
      for (int h = 0; h < HP / 2; h++) amm_unpack2(t2[h], t[2 * h], t[2 * h + 1]);
      __syncwarp();      // every lane has read the row's raw scores before the mixed ones overwrite them
#pragma unroll
      for (int h = 0; h < HP; h++)
        if (h < H) row[h * AMM_SLOT + lane] = seen ? t[h] : AMX_NEG;
      __syncwarp();
      if (lane < H) {      // head `lane`: its 32 scores of the row, the streaming softmax in registers
        float4* mine = reinterpret_cast<float4*>(row + lane * AMM_SLOT);
        float v[AMM_KT];
#pragma unroll
        for (int x = 0; x < AMM_KT / 4; x++) {
          const float4 f = mine[x];
          v[4 * x] = f.x; v[4 * x + 1] = f.y; v[4 * x + 2] = f.z; v[4 * x + 3] = f.w;
        }
        float tmax = v[0];
#pragma unroll
        for (int x = 1; x < AMM_KT; x++) tmax = fmaxf(tmax, v[x]);
        const float m_new = fmaxf(m_run, tmax);
        const float corr = amm_exp2(m_run - m_new);      // 1 while nothing was seen (both at the floor)
        const float m_use = m_new > 0.5f * AMX_NEG ? m_new : 0.f;      // nothing seen yet: every weight is 2^(floor) = 0
        float sum = 0.f;
        uint32_t hi[AMM_KT / 2], lo[AMM_KT / 2];
#pragma unroll
        for (int x = 0; x < AMM_KT; x += 2) {
          const float w0 = amm_exp2(v[x] - m_use);
          const float w1 = amm_exp2(v[x + 1] - m_use);
          sum += w0 + w1;
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(w0, w1);
          const __nv_bfloat162 l2 = __floats2bfloat162_rn(w0 - __low2float(h2), w1 - __high2float(h2));
          hi[x / 2] = *reinterpret_cast<const uint32_t*>(&h2);
          lo[x / 2] = *reinterpret_cast<const uint32_t*>(&l2);
        }
        l_run = l_run * corr + sum;
        m_run = m_new;
        corr_s[lane * AMM_ROWS + i] = corr;
        uint4* dst = reinterpret_cast<uint4*>(mine);
#pragma unroll
        for (int x = 0; x < AMM_KT / 8; x++) {
          dst[x] = make_uint4(hi[4 * x], hi[4 * x + 1], hi[4 * x + 2], hi[4 * x + 3]);
          dst[AMM_KT / 8 + x] = make_uint4(lo[4 * x], lo[4 * x + 1], lo[4 * x + 2], lo[4 * x + 3]);
        }
      }
    }
    // the values [c][d][j], zero where no position is yet
#pragma unroll
    for (int x = 0; x < VPT; x++) {
      const int idx = threadIdx.x + x * blockDim.x;
      if (idx < v_total) {
        const int cd = idx / (AMM_KT / 8), ch = idx - cd * (AMM_KT / 8);
        uint4 v = vreg[x];
        const int left = kv_len - (key0 + ch * 8);      // positions of this piece that exist
        if (left < 8) {
          bf16* e = reinterpret_cast<bf16*>(&v);
#pragma unroll
          for (int y = 0; y < 8; y++)
            if (y >= left) e[y] = __float2bfloat16_rn(0.f);
        }
        *reinterpret_cast<uint4*>(kv_s + (size_t)cd * VS + ch * 8) = v;
      }
    }
    __syncthreads();
    if (k_ahead && ut + 1 < n_tiles) {      // the next tile's keys on their way
      const int nkey0 = key0 + AMM_KT;
      const int npage = block_table[(size_t)b * bt_width + nkey0 / page_size];
      const int nin = nkey0 % page_size;
#pragma unroll
      for (int x = 0; x < KPT; x++) {
        const int idx = threadIdx.x + x * blockDim.x;
        kreg[x] = make_uint4(0, 0, 0, 0);
        if (idx < k_total) {
          const int cj = idx / k_per_row, d0 = (idx - cj * k_per_row) * 8;
          const int c = cj / AMM_KT, j = cj - c * AMM_KT;
          if (npage >= 0 && nkey0 + j < kv_len)
            kreg[x] = *reinterpret_cast<const uint4*>(k_pool + (((size_t)npage * G + c) * page_size + nin + j) * hd + d0);
        }
      }
    }
    // 3. weighted values: units (head h, 8 dimensions dt)
#pragma unroll
    for (int uu = 0; uu < UPW; uu++) {
      const int u = warp + uu * AMM_WARPS;
      if (u >= n_units) break;
      const int h = u / n_dt, dt = u - h * n_dt;
      const float c0 = corr_s[h * AMM_ROWS + gid], c1 = corr_s[h * AMM_ROWS + gid + 8];
      acc[uu][0] *= c0;
      acc[uu][1] *= c0;
      acc[uu][2] *= c1;
      acc[uu][3] *= c1;
      // a lane's rows of the weights: row (lane % 16), the 8 keys from 8 * (lane / 16) on; hi at bytes 0.., lo at 64..
      const unsigned char* pa = reinterpret_cast<const unsigned char*>(raw_s + (size_t)(lane & 15) * RS + h * AMM_SLOT) + 16 * (lane >> 4);
      const bf16* vb = kv_s + ((size_t)(h / Gq) * vd + dt * 8 + (lane & 7)) * VS + 8 * ((lane >> 3) & 1);
#pragma unroll
      for (int k0 = 0; k0 < AMM_KT; k0 += 16) {
        uint32_t b0, b1, a[4];
        amm_ldsm2(b0, b1, vb + k0);
        amm_ldsm4(a, pa + 2 * k0);
        amm_mma(acc[uu], a, b0, b1);
        amm_ldsm4(a, pa + 64 + 2 * k0);
        amm_mma(acc[uu], a, b0, b1);
      }
    }
  }
  // the sums of every (head, row) to where the units' threads find them
  __syncthreads();
  if (lane < H) corr_s[lane * AMM_ROWS + warp] = l_run > 0.f ? 1.0f / l_run : 0.f;
  __syncthreads();
#pragma unroll
  for (int uu = 0; uu < UPW; uu++) {
    const int u = warp + uu * AMM_WARPS;
    if (u >= n_units) break;
    const int h = u / n_dt, dt = u - h * n_dt;
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const int i = gid + 8 * half;
      if (i >= nrows) continue;
      const size_t m = (size_t)q0 + row_lo + i;
      const float inv = corr_s[h * AMM_ROWS + i];
      const int d = dt * 8 + 2 * tig;
      float o0 = acc[uu][2 * half] * inv, o1 = acc[uu][2 * half + 1] * inv;
      if (gate) {
        const float* gp = gate + m * ldg + (size_t)h * vd + d;
        o0 *= 1.0f / (1.0f + expf(-gp[0]));
        o1 *= 1.0f / (1.0f + expf(-gp[1]));
      }
      *reinterpret_cast<__nv_bfloat162*>(out + (m * H + h) * vd + d) = __floats2bfloat162_rn(o0, o1);
    }
  }
}

static size_t amm_smem(int H, int HP, int G, int hd, int vd) {
  const size_t kv = (size_t)G * (size_t)max(AMM_KT * (hd + 8), vd * (AMM_KT + 8));
  return sizeof(float) * ((size_t)H * HP + (size_t)H * AMM_ROWS + (size_t)AMM_ROWS * (H * AMM_SLOT + AMM_ROW_PAD)) +
         2 * ((size_t)H * AMM_ROWS * (hd + 8) + kv);
}

// Whether the tensor-core kernel takes these sizes (bfloat16 prompts).
LEB_API int leb_attention_mixed_mma_supported(int H, int G, int hd, int vd, int page_size) {
  if (H < 1 || H > 32 || G < 1 || H % G || hd % 16 || hd < 16 || vd % 8 || vd < 8 || page_size % AMM_KT) return 0;
  if (H * (vd / 8) > 16 * AMM_WARPS) return 0;          // a thread holds at most 16 units' sums
  if (G * vd * (AMM_KT / 8) > 4 * 32 * AMM_WARPS) return 0;      // the values of a tile in four pieces a thread
  const int HP = H <= 4 ? 4 : H <= 8 ? 8 : H <= 16 ? 16 : 32;
  return amm_smem(H, HP, G, hd, vd) <= 227 * 1024 ? 1 : 0;
}

LEB_API int leb_attention_mixed_mma(void* out, const void* q, int ldq, const void* k_pool, const void* v_pool,
                                    const int* block_table, int bt_width, const int* seq_slot, const int* seq_pos0,
                                    const int* seq_qstart, const int* seq_qlen, const float* talk, const float* gate, int ldg,
                                    int M, int B, int H, int G, int hd, int vd, int page_size, int window, float scale,
                                    int max_qlen, cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(leb_attention_mixed_mma_supported(H, G, hd, vd, page_size), "leb_attention_mixed_mma: sizes %d/%d heads of %d/%d not taken", H, G, hd, vd);
  LEB_REQUIRE(ldq % 8 == 0 && ((uintptr_t)q & 15) == 0, "leb_attention_mixed_mma: query rows must start on 16 bytes");
  LEB_REQUIRE(B <= 65535, "leb_attention_mixed_mma: step too large");
  const int HP = H <= 4 ? 4 : H <= 8 ? 8 : H <= 16 ? 16 : 32;
  const size_t smem = amm_smem(H, HP, G, hd, vd);
  const int units = H * (vd / 8);
  int upw = ceil_div(units, AMM_WARPS);
  upw = upw <= 1 ? 1 : upw <= 2 ? 2 : upw <= 4 ? 4 : upw <= 8 ? 8 : 16;
  const dim3 grid(ceil_div(max_qlen, AMM_ROWS), B), block(32 * AMM_WARPS);
  const bool ahead = upw <= 8 && HP <= 16 && G * AMM_KT * (hd / 8) <= 4 * 32 * AMM_WARPS;
  LebPlainLaunches plain(true);
#define AMM_LAUNCH(HP_, UPW_) { if (ahead) AMM_LAUNCH2(HP_, UPW_, true) else AMM_LAUNCH2(HP_, UPW_, false) }
#define AMM_LAUNCH2(HP_, UPW_, AH_)                                                                                        \
  {                                                                                                                        \
    static size_t set = 48 * 1024;                                                                                         \
    if (smem > set) {                                                                                                      \
      if (cudaFuncSetAttribute(attention_mixed_mma_kernel<HP_, UPW_, AH_>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                               (int)smem) != cudaSuccess)                                                                  \
        return leb_fail("leb_attention_mixed_mma: %zu bytes of shared memory per block refused", smem);                   \
      set = smem;                                                                                                          \
    }                                                                                                                      \
    leb_launch(attention_mixed_mma_kernel<HP_, UPW_, AH_>, grid, block, smem, st, (bf16*)out, (const bf16*)q, ldq,         \
               (const bf16*)k_pool, (const bf16*)v_pool, block_table, bt_width, seq_slot, seq_pos0, seq_qstart, seq_qlen,  \
               talk, gate, ldg, H, G, hd, vd, page_size, window, scale);                                                   \
  }
#define AMM_UPW(HP_)                            \
  {                                             \
    if (upw == 1) AMM_LAUNCH(HP_, 1)            \
    else if (upw == 2) AMM_LAUNCH(HP_, 2)       \
    else if (upw == 4) AMM_LAUNCH(HP_, 4)       \
    else if (upw == 8) AMM_LAUNCH(HP_, 8)       \
    else AMM_LAUNCH(HP_, 16)                    \
  }
  if (HP == 4) AMM_UPW(4)
  else if (HP == 8) AMM_UPW(8)
  else if (HP == 16) AMM_UPW(16)
  else AMM_UPW(32)
#undef AMM_UPW
#undef AMM_LAUNCH
#undef AMM_LAUNCH2
  LEB_CHECK_LAUNCH("leb_attention_mixed_mma");
  return 0;
}

// Bytes of shared memory a block needs for the given shape.
static size_t amx_smem(int H, int G, int hd, int vd, int QT, int KT, size_t esz) {
  const int EV = (int)(16 / esz);
  const int hdp = (hd + 7) & ~7, vdp = (vd + 7) & ~7, NP = QT * H;
  return sizeof(float) * (size_t)(((H * H + 3) & ~3) + NP * hdp + 2 * NP * KT) + esz * (size_t)G * KT * (hdp + EV + vdp);
}

// out [M, H*vd] and q [M, H*hd] (row stride ldq) in the cache's type; part: float scratch of
// M*H*n_splits*(vd+2) when n_splits > 1; talk [H, H] float; gate float [M, H*vd] with row stride ldg, or null.
LEB_API int leb_attention_mixed(void* out, float* part, const void* q, int ldq, const void* k_pool, const void* v_pool,
                                int dtype, const int* block_table, int bt_width, const int* seq_slot, const int* seq_pos0,
                                const int* seq_qstart, const int* seq_qlen, const float* talk, const float* gate, int ldg,
                                int M, int B, int H, int G, int hd, int vd, int page_size, int window, float scale,
                                int max_qlen, int n_splits, cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(H >= 1 && G >= 1 && H % G == 0, "leb_attention_mixed: %d heads do not divide into %d kv heads", H, G);
  LEB_REQUIRE(H <= 128, "leb_attention_mixed: %d heads (a block mixes all heads of a row: up to 128)", H);
  LEB_REQUIRE(hd >= 1 && hd <= 512 && vd >= 1 && vd <= 256, "leb_attention_mixed: head sizes %d / %d (up to 512 / 256)", hd, vd);
  LEB_REQUIRE(page_size % 32 == 0, "leb_attention_mixed: pages of %d positions", page_size);
  LEB_REQUIRE(n_splits >= 1 && (n_splits == 1 || part), "leb_attention_mixed: %d splits need scratch", n_splits);
  LEB_REQUIRE(B <= 65535 && n_splits <= 65535, "leb_attention_mixed: step too large");
  LEB_REQUIRE(dtype == LEB_F32 || dtype == LEB_BF16, "leb_attention_mixed: unknown dtype %d", dtype);
  const size_t esz = dtype == LEB_BF16 ? 2 : 4;
  // rows of a block: up to 128 (row, head) pairs, fewer when a sequence brings fewer rows; keys of a tile: 32, or
  // fewer where the tiles of all kv heads would not fit
  const size_t room = 200 * 1024;
  int QT = max(1, min(max_qlen, min(16, 128 / H)));
  int KT = 32;
  while (amx_smem(H, G, hd, vd, QT, KT, esz) > room && QT > 1) QT = (QT + 1) / 2;
  while (amx_smem(H, G, hd, vd, QT, KT, esz) > room && KT > 8) KT /= 2;
  const size_t smem = amx_smem(H, G, hd, vd, QT, KT, esz);
  LEB_REQUIRE(smem <= 227 * 1024, "leb_attention_mixed: %d kv heads of %d / %d do not fit shared memory", G, hd, vd);
  const int NP = QT * H;
  int warps = min(AMX_MAX_WARPS, max(4, NP));
  int rpw = ceil_div(NP, warps);
  rpw = rpw <= 1 ? 1 : rpw <= 2 ? 2 : rpw <= 4 ? 4 : 8;
  warps = max(4, min(AMX_MAX_WARPS, ceil_div(NP, rpw)));
  const int hdl = ceil_div(vd, 32);
  const dim3 grid(ceil_div(max_qlen, QT), n_splits, B), block(32 * warps);
  LebPlainLaunches plain(true);
#define AMX_LAUNCH(T_, HDL_, RPW_)                                                                                          \
  {                                                                                                                         \
    static size_t set = 48 * 1024;                                                                                          \
    if (smem > set) {                                                                                                       \
      if (cudaFuncSetAttribute(attention_mixed_kernel<T_, HDL_, RPW_>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                               (int)smem) != cudaSuccess)                                                                   \
        return leb_fail("leb_attention_mixed: %zu bytes of shared memory per block refused", smem);                        \
      set = smem;                                                                                                           \
    }                                                                                                                       \
    leb_launch(attention_mixed_kernel<T_, HDL_, RPW_>, grid, block, smem, st, (T_*)out, part, (const T_*)q, ldq,            \
               (const T_*)k_pool, (const T_*)v_pool, block_table, bt_width, seq_slot, seq_pos0, seq_qstart, seq_qlen, talk, \
               gate, ldg, H, G, hd, vd, page_size, window, scale, QT, KT, n_splits);                                        \
  }
#define AMX_RPW(T_, HDL_)                       \
  {                                             \
    if (rpw == 1) AMX_LAUNCH(T_, HDL_, 1)       \
    else if (rpw == 2) AMX_LAUNCH(T_, HDL_, 2)  \
    else if (rpw == 4) AMX_LAUNCH(T_, HDL_, 4)  \
    else AMX_LAUNCH(T_, HDL_, 8)                \
  }
#define AMX_HDL(T_)                             \
  {                                             \
    if (hdl <= 1) AMX_RPW(T_, 1)                \
    else if (hdl <= 2) AMX_RPW(T_, 2)           \
    else if (hdl <= 4) AMX_RPW(T_, 4)           \
    else AMX_RPW(T_, 8)                         \
  }
  if (dtype == LEB_F32) AMX_HDL(float)
  else AMX_HDL(bf16)
#undef AMX_HDL
#undef AMX_RPW
#undef AMX_LAUNCH
  LEB_CHECK_LAUNCH("leb_attention_mixed");
  if (n_splits > 1) {
    const size_t pairs = (size_t)M * H;
    const dim3 mgrid((unsigned)((pairs + 3) / 4)), mblock(128);
    if (dtype == LEB_F32)
      leb_launch(attention_mixed_merge_kernel<float>, mgrid, mblock, 0, st, (float*)out, part, gate, ldg, pairs, H, vd, n_splits);
    else
      leb_launch(attention_mixed_merge_kernel<bf16>, mgrid, mblock, 0, st, (bf16*)out, part, gate, ldg, pairs, H, vd, n_splits);
    LEB_CHECK_LAUNCH("leb_attention_mixed (merge)");
  }
  return 0;
}
