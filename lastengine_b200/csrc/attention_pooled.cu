// Attention inside a sliding window with pooled blocks behind it, over the paged cache, for packed
// rows of several sequences: the general kernels (any head sizes up to 256, float or bfloat16 cache).
//
// Position i sees the positions j with 0 <= i - j < window, and one pooled key and value for every
// block of `pool` positions that lies wholly before the window: block b = [b pool, b pool + pool - 1] is
// seen when b pool + pool - 1 <= i - window, i.e. the first nb(i) = max(0, i - window + 1) / pool blocks.
// A pooled key is the mean of the block's keys as the cache holds them (after norm and rotation), a
// pooled value the mean of its cached values.  Positions that left the window and whose block is not
// complete are seen by nobody.  Positions and pooled blocks share one softmax.  score = (q . k) times a
// number per head (the configured scale times the head's learned temperature).
//
// Values are cached rotated: the value of position j is turned by j over all of its width (pairs
// m, m + vd/2; pair m by j * freq[m]) before it is stored, and a head's result at position i is turned
// back by -i before it leaves the kernel (whole or merged from the splits).
//
// Three entry points: the rows' preparation (bias, per-head RMS norm with a weight, rotation of q and k,
// rotation of v, cache write), the pooled rows of the blocks a step completes (read back from the
// cache, so they do not depend on how the sequence was cut into steps), and the attention itself with
// the merge of its key-range splits (decode steps).  Scores, softmax, sums and rotations are float.
#include "common.cuh"

#define PAT_WARPS 4
#define PAT_RPW 8
#define PAT_NEG (-1e30f)

// ---- preparation ---------------------------------------------------------------------------------
// proj [M, ldp] float: q heads | k heads | v heads as the projection left them; bias [same columns] or null.
template <typename T>
__global__ void __launch_bounds__(32 * PAT_WARPS)
pooled_prep_kernel(T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool, const float* __restrict__ proj,
                   int ldp, const float* __restrict__ bias, const float* __restrict__ qw, const float* __restrict__ kw,
                   float eps, const float* __restrict__ freq_qk, int rot, const float* __restrict__ freq_v,
                   const int* __restrict__ block_table, int bt_width, const int* __restrict__ row_seq,
                   const int* __restrict__ row_pos, const int* __restrict__ seq_slot, int nh, int nkv, int hd, int vd,
                   int page_size) {
  extern __shared__ float buf_all[];
  pdl_wait();
  const size_t m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wmax = hd > vd ? hd : vd;
  float* buf = buf_all + (size_t)warp * wmax;
  const int b = row_seq[m];
  const int slot = seq_slot[b];
  const int pos = row_pos[m];
  const int page = slot >= 0 ? block_table[(size_t)b * bt_width + pos / page_size] : -1;
  const int in_page = pos % page_size;
  const float fpos = (float)pos;
  {      // a warp a head: blockIdx.y counts blocks of PAT_WARPS heads of q | k | v
    const int hh = blockIdx.y * PAT_WARPS + warp;
    if (hh >= nh + 2 * nkv) return;
    const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
    const int width = (is_q || is_k) ? hd : vd;
    const int col = is_q ? hh * hd : (is_k ? nh * hd + (hh - nh) * hd : (nh + nkv) * hd + (hh - nh - nkv) * vd);
    const float* src = proj + m * ldp + col;
    float ss = 0.f;
    for (int i = lane; i < width; i += 32) {
      const float x = src[i] + (bias ? bias[col + i] : 0.f);
      buf[i] = x;
      ss += x * x;
    }
    __syncwarp();
    int nrot;
    const float* freq;
    if (is_q || is_k) {
      ss = warp_sum(ss);
      const float r = 1.0f / sqrtf(ss / (float)hd + eps);
      const float* w = is_q ? qw : kw;
      for (int i = lane; i < width; i += 32) buf[i] = buf[i] * r * (w ? w[i] : 1.0f);
      __syncwarp();
      nrot = rot;
      freq = freq_qk;
    } else {
      nrot = vd;
      freq = freq_v;
    }
    if (!freq) nrot = 0;
    const int half = nrot / 2;
    auto put = [&](int i, float val) {
      if (is_q) {
        q_out[(m * nh + hh) * hd + i] = from_f32<T>(val);
      } else if (page >= 0) {
        if (is_k) k_pool[(((size_t)page * nkv + (hh - nh)) * page_size + in_page) * hd + i] = from_f32<T>(val);
        else v_pool[(((size_t)page * nkv + (hh - nh - nkv)) * vd + i) * page_size + in_page] = from_f32<T>(val);
      }
    };
    for (int i = lane; i < half; i += 32) {      // a pair (i, i + half) shares its angle
      float sn, cs;
      sincosf(fpos * freq[i], &sn, &cs);
      const float lo = buf[i], hi = buf[i + half];
      put(i, lo * cs - hi * sn);
      put(i + half, hi * cs + lo * sn);
    }
    for (int i = nrot + lane; i < width; i += 32) put(i, buf[i]);
    __syncwarp();
  }
}

LEB_API int leb_pooled_attn_prep(void* q_out, void* k_pool, void* v_pool, int dtype, const float* proj, int ldp,
                                 const float* bias, const float* qw, const float* kw, float eps, const float* freq_qk,
                                 int rot, const float* freq_v, const int* block_table, int bt_width, const int* row_seq,
                                 const int* row_pos, const int* seq_slot, int M, int nh, int nkv, int hd, int vd,
                                 int page_size, cudaStream_t st) {
  if (M <= 0) return 0;
  LEB_REQUIRE(hd >= 1 && hd <= 256 && vd >= 1 && vd <= 256, "leb_pooled_attn_prep: head sizes %d / %d outside 1..256", hd, vd);
  LEB_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0 && vd % 2 == 0, "leb_pooled_attn_prep: rotated widths must be even (%d, %d)", rot, vd);
  const size_t smem = (size_t)PAT_WARPS * (hd > vd ? hd : vd) * sizeof(float);
  const dim3 grid(M, ceil_div(nh + 2 * nkv, PAT_WARPS));
  LEB_REQUIRE(grid.y <= 65535, "leb_pooled_attn_prep: %d heads in a row", nh + 2 * nkv);
  LebPlainLaunches plain(true);
  if (dtype == LEB_F32)
    leb_launch(pooled_prep_kernel<float>, grid, dim3(32 * PAT_WARPS), smem, st, (float*)q_out, (float*)k_pool, (float*)v_pool,
               proj, ldp, bias, qw, kw, eps, freq_qk, rot, freq_v, block_table, bt_width, row_seq, row_pos, seq_slot, nh, nkv,
               hd, vd, page_size);
  else if (dtype == LEB_BF16)
    leb_launch(pooled_prep_kernel<bf16>, grid, dim3(32 * PAT_WARPS), smem, st, (bf16*)q_out, (bf16*)k_pool, (bf16*)v_pool,
               proj, ldp, bias, qw, kw, eps, freq_qk, rot, freq_v, block_table, bt_width, row_seq, row_pos, seq_slot, nh, nkv,
               hd, vd, page_size);
  else
    return leb_fail("leb_pooled_attn_prep: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_pooled_attn_prep");
  return 0;
}

// ---- pooled rows of the blocks this step completes -------------------------------------------------
// Block (x, kv head, sequence): pooled block floor(pos0 / pool) + x, if its last position lies among the
// step's rows.  The `pool` cached keys (values) are added in the order of their positions and divided by pool.
template <typename T>
__global__ void __launch_bounds__(128)
pool_blocks_kernel(T* __restrict__ pk_pool, T* __restrict__ pv_pool, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                   const int* __restrict__ block_table, int bt_width, const int* __restrict__ pool_table, int pt_width,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_pos0, const int* __restrict__ seq_qlen,
                   int nkv, int hd, int vd, int page_size, int pool) {
  pdl_wait();
  const int b = blockIdx.z, kvh = blockIdx.y;
  if (seq_slot[b] < 0) return;
  const int pos0 = seq_pos0[b], n = seq_qlen ? seq_qlen[b] : 1;
  const int blk = pos0 / pool + blockIdx.x;
  const int last = blk * pool + pool - 1;
  if (last < pos0 || last >= pos0 + n) return;
  const int ppage = pool_table[(size_t)b * pt_width + blk / page_size];
  if (ppage < 0) return;
  const int pin = blk % page_size;
  const float inv = 1.0f / (float)pool;
  for (int i = threadIdx.x; i < hd + vd; i += blockDim.x) {
    // one address form for a key's number and a value's, so that the loads carry no branch and eight are in flight
    const bool is_k = i < hd;
    const T* src = is_k ? k_pool + i : v_pool + (size_t)(i - hd) * page_size;
    const size_t page_step = (size_t)nkv * page_size * (is_k ? hd : vd);
    const size_t head_at = (size_t)kvh * page_size * (is_k ? hd : vd);
    const int pos_step = is_k ? hd : 1;
    float s = 0.f;
    for (int j0 = 0; j0 < pool; j0 += 8) {      // added in the order of the positions
      int page[8];
#pragma unroll
      for (int u = 0; u < 8; u++)
        page[u] = j0 + u < pool ? block_table[(size_t)b * bt_width + (blk * pool + j0 + u) / page_size] : -1;
      float t[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int in_page = (blk * pool + j0 + u) % page_size;
        t[u] = to_f32(src[(size_t)max(page[u], 0) * page_step + head_at + (size_t)in_page * pos_step]);
      }
#pragma unroll
      for (int u = 0; u < 8; u++) s += page[u] >= 0 ? t[u] : 0.f;
    }
    if (i < hd) pk_pool[(((size_t)ppage * nkv + kvh) * page_size + pin) * hd + i] = from_f32<T>(s * inv);
    else pv_pool[(((size_t)ppage * nkv + kvh) * vd + (i - hd)) * page_size + pin] = from_f32<T>(s * inv);
  }
}

LEB_API int leb_pool_blocks(void* pk_pool, void* pv_pool, const void* k_pool, const void* v_pool, int dtype,
                            const int* block_table, int bt_width, const int* pool_table, int pt_width, const int* seq_slot,
                            const int* seq_pos0, const int* seq_qlen, int B, int max_qlen, int nkv, int hd, int vd,
                            int page_size, int pool, cudaStream_t st) {
  if (B <= 0 || max_qlen <= 0) return 0;
  LEB_REQUIRE(pool >= 1, "leb_pool_blocks: blocks of %d positions", pool);
  const dim3 grid(ceil_div(max_qlen, pool) + 1, nkv, B), block(128);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_pool_blocks: grid too large");
  LebPlainLaunches plain(true);
  if (dtype == LEB_F32)
    leb_launch(pool_blocks_kernel<float>, grid, block, 0, st, (float*)pk_pool, (float*)pv_pool, (const float*)k_pool,
               (const float*)v_pool, block_table, bt_width, pool_table, pt_width, seq_slot, seq_pos0, seq_qlen, nkv, hd, vd,
               page_size, pool);
  else if (dtype == LEB_BF16)
    leb_launch(pool_blocks_kernel<bf16>, grid, block, 0, st, (bf16*)pk_pool, (bf16*)pv_pool, (const bf16*)k_pool,
               (const bf16*)v_pool, block_table, bt_width, pool_table, pt_width, seq_slot, seq_pos0, seq_qlen, nkv, hd, vd,
               page_size, pool);
  else
    return leb_fail("leb_pool_blocks: unknown dtype %d", dtype);
  LEB_CHECK_LAUNCH("leb_pool_blocks");
  return 0;
}

// ---- attention -------------------------------------------------------------------------------------
// Block = 4 warps: one sequence, one kv head, a chunk of HC <= 8 of its query heads, QT rows (QT*HC <= 32
// query vectors) and one split of the tile range.  The tile range is the pooled tiles (32 pooled blocks
// each, from the pooled pools) followed by the window's tiles (32 positions each, from the cache); per
// tile lane = key for q.k and lane = dimension for p.v, with one running (max, sum, acc) over both kinds.
__device__ __forceinline__ int blocks_seen(int qpos, int window, int pool) {
  const int past = qpos - window + 1;
  return (window > 0 && pool > 0 && past > 0) ? past / pool : 0;
}

// Value heads up to 64 wide keep four blocks on an SM (128 registers a thread): the grids of a decode step are
// sized for that many, and a block more than fit waits for a place.
template <typename T, typename CT, int HDL>
__global__ void __launch_bounds__(32 * PAT_WARPS, HDL <= 2 ? 4 : 1)
attention_pooled_kernel(T* __restrict__ out, float* __restrict__ part, const T* __restrict__ q,
                        const CT* __restrict__ k_pool, const CT* __restrict__ v_pool, const int* __restrict__ block_table,
                        int bt_width, const CT* __restrict__ pk_pool, const CT* __restrict__ pv_pool,
                        const int* __restrict__ pool_table, int pt_width, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_pos0, const int* __restrict__ seq_qstart, const int* __restrict__ seq_qlen,
                        const float* __restrict__ head_scale, const float* __restrict__ freq_v, int nh, int nkv, int hd,
                        int vd, int page_size, int window, int pool, int QT, int HC, int n_splits) {
  extern __shared__ __align__(16) float sm[];
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = nh / nkv;
  const int n_hc = (G + HC - 1) / HC;
  const int kvh = blockIdx.y / n_hc, hc = blockIdx.y % n_hc;
  const int b = blockIdx.z / n_splits, split = blockIdx.z % n_splits;
  const int slot = seq_slot[b];
  const int qlen = seq_qlen ? seq_qlen[b] : 1;
  const int row_lo = blockIdx.x * QT;
  if (row_lo >= qlen) return;
  const int nrows = min(QT, qlen - row_lo);
  const int nheads = min(HC, G - hc * HC);
  const int q0 = seq_qstart[b];
  const int pos0 = seq_pos0[b];
  const int R = QT * HC;
  const int KS = ((hd + 3) & ~3) + 4;      // a key's row: 16-byte pieces, and eight lanes' pieces fall in 32 different banks
  constexpr int VS = 36;                    // a value dimension's row of 32 positions, likewise
  const bool hd4 = hd % 4 == 0;

  float* q_s = sm;                 // [R][hd]
  float* k_s = q_s + ((R * hd + 3) & ~3);   // [32][KS], on 16 bytes like everything behind it
  float* v_s = k_s + 32 * KS;      // [vd][VS]: a dimension's 32 positions of the tile
  float* p_s = v_s + VS * vd;      // [PAT_WARPS][32]
  float* o_s = p_s + PAT_WARPS * 32;   // [PAT_WARPS][vd]

  if (slot < 0) {  // padding sequence: defined output, no cache access
    for (int r = warp; r < R; r += PAT_WARPS) {
      const int i = r / HC, j = r % HC;
      if (i >= nrows || j >= nheads) continue;
      const int h = kvh * G + hc * HC + j;
      const size_t m = (size_t)q0 + row_lo + i;
      if (n_splits == 1) {
        for (int d = lane; d < vd; d += 32) out[(m * nh + h) * vd + d] = from_f32<T>(0.f);
      } else {
        float* pp = part + ((m * nh + h) * n_splits + split) * (size_t)(vd + 2);
        if (lane == 0) { pp[0] = PAT_NEG; pp[1] = 0.f; }
        for (int d = lane; d < vd; d += 32) pp[2 + d] = 0.f;
      }
    }
    return;
  }

  for (int idx = threadIdx.x; idx < R * hd; idx += blockDim.x) {
    const int r = idx / hd, d = idx - r * hd;
    const int i = r / HC, j = r % HC;
    float v = 0.f;
    if (i < nrows && j < nheads) {
      const int h = kvh * G + hc * HC + j;
      v = to_f32(q[((size_t)(q0 + row_lo + i) * nh + h) * hd + d]);
    }
    q_s[idx] = v;
  }

  const int kv_len = pos0 + qlen;
  const int pos_lo = pos0 + row_lo, pos_hi = pos0 + row_lo + nrows - 1;
  const int key_lo = (window > 0 && pos_lo + 1 > window) ? pos_lo + 1 - window : 0;
  const int tile_first = key_lo / 32, tile_last = pos_hi / 32;
  const int nb_hi = blocks_seen(pos_hi, window, pool);     // pooled blocks the block's last row sees
  const int np_tiles = (nb_hi + 31) / 32;
  const int n_tiles = np_tiles + tile_last - tile_first + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int t_lo = split * per_split;
  const int t_hi = min(n_tiles, t_lo + per_split);

  float mx[PAT_RPW], l[PAT_RPW], acc[PAT_RPW][HDL];
#pragma unroll
  for (int ri = 0; ri < PAT_RPW; ri++) {
    mx[ri] = PAT_NEG;
    l[ri] = 0.f;
#pragma unroll
    for (int jj = 0; jj < HDL; jj++) acc[ri][jj] = 0.f;
  }

  constexpr int EV = 16 / (int)sizeof(CT);      // cached numbers in a 16-byte load
  // A tile's keys are one contiguous run and a dimension's 32 values another, so 16-byte loads bring a tile in.
  // When two of each kind per thread cover a tile, the next tile's loads are issued before this tile is
  // computed and stored to shared memory after it: the walk over the tiles does not wait on global memory.
  const int nvk = 32 * hd / EV, nvv = vd * (32 / EV);
  const bool vec = hd % EV == 0;
  const bool ahead = vec && max(nvk, nvv) <= 2 * (int)blockDim.x;
  struct Tile { bool pooled; int key0, limit, page; const CT *kp, *vp; size_t base, vbase; };
  auto tile_of = [&](int ut) {
    Tile t;
    t.pooled = ut < np_tiles;
    t.key0 = t.pooled ? ut * 32 : (tile_first + ut - np_tiles) * 32;
    t.limit = t.pooled ? nb_hi : kv_len;          // rows beyond it hold stale bits
    t.page = t.pooled ? pool_table[(size_t)b * pt_width + t.key0 / page_size]
                      : block_table[(size_t)b * bt_width + t.key0 / page_size];
    t.kp = t.pooled ? pk_pool : k_pool;
    t.vp = t.pooled ? pv_pool : v_pool;
    t.base = (((size_t)(t.page < 0 ? 0 : t.page) * nkv + kvh) * page_size + t.key0 % page_size) * hd;
    t.vbase = ((size_t)(t.page < 0 ? 0 : t.page) * nkv + kvh) * vd * page_size + t.key0 % page_size;
    return t;
  };
  auto load16 = [&](const Tile& t, int i0, uint4* rk, uint4* rv) {
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const int idx = i0 + u * blockDim.x + threadIdx.x;
      rk[u] = make_uint4(0, 0, 0, 0);
      rv[u] = make_uint4(0, 0, 0, 0);
      if (t.page >= 0 && idx < nvk && t.key0 + idx * EV / hd < t.limit)
        rk[u] = *reinterpret_cast<const uint4*>(t.kp + t.base + (size_t)idx * EV);
      if (t.page >= 0 && idx < nvv)
        rv[u] = *reinterpret_cast<const uint4*>(t.vp + t.vbase + (size_t)(idx / (32 / EV)) * page_size + (idx % (32 / EV)) * EV);
    }
  };
  auto store16 = [&](const Tile& t, int i0, const uint4* rk, const uint4* rv) {
#pragma unroll
    for (int u = 0; u < 2; u++) {
      const int idx = i0 + u * blockDim.x + threadIdx.x;
      if (idx < nvk) {
        const int kk = idx * EV / hd, d = idx * EV - kk * hd;
        const CT* el = reinterpret_cast<const CT*>(&rk[u]);
#pragma unroll
        for (int j = 0; j < EV; j++) k_s[kk * KS + d + j] = to_f32(el[j]);
      }
      if (idx < nvv) {
        const int d = idx / (32 / EV), k0 = (idx % (32 / EV)) * EV;
        const CT* el = reinterpret_cast<const CT*>(&rv[u]);
#pragma unroll
        for (int j = 0; j < EV; j++) v_s[d * VS + k0 + j] = (t.key0 + k0 + j < t.limit) ? to_f32(el[j]) : 0.f;
      }
    }
  };
  uint4 nk[2], nv[2];      // the tile ahead
  Tile tnext;
  if (ahead && t_lo < t_hi) {
    tnext = tile_of(t_lo);
    load16(tnext, 0, nk, nv);
  }
  for (int ut = t_lo; ut < t_hi; ut++) {
    const Tile tl = ahead ? tnext : tile_of(ut);
    const bool pooled = tl.pooled;
    const int key0 = tl.key0;
    __syncthreads();
    if (ahead) {
      store16(tl, 0, nk, nv);
    } else if (vec) {
      for (int i0 = 0; i0 < max(nvk, nvv); i0 += 2 * blockDim.x) {
        uint4 rk[2], rv[2];
        load16(tl, i0, rk, rv);
        store16(tl, i0, rk, rv);
      }
    } else {
      for (int idx = threadIdx.x; idx < 32 * hd; idx += blockDim.x) {
        const int kk = idx / hd, d = idx - kk * hd;
        float kv = 0.f;
        if (tl.page >= 0 && key0 + kk < tl.limit) kv = to_f32(tl.kp[tl.base + idx]);
        k_s[kk * KS + d] = kv;
      }
      for (int idx = threadIdx.x; idx < 32 * vd; idx += blockDim.x) {
        const int d = idx / 32, kk = idx - d * 32;
        float vv = 0.f;
        if (tl.page >= 0 && key0 + kk < tl.limit) vv = to_f32(tl.vp[tl.vbase + (size_t)d * page_size + kk]);
        v_s[d * VS + kk] = vv;
      }
    }
    __syncthreads();
    if (ahead && ut + 1 < t_hi) {
      tnext = tile_of(ut + 1);
      load16(tnext, 0, nk, nv);
    }
#pragma unroll
    for (int ri = 0; ri < PAT_RPW; ri++) {
      const int r = warp + ri * PAT_WARPS;
      if (r >= R) break;
      const int i = r / HC, j = r % HC;
      if (i >= nrows || j >= nheads) continue;
      const int qpos = pos0 + row_lo + i;
      const int h = kvh * G + hc * HC + j;
      const float* qv = q_s + r * hd;
      const float* kr = k_s + lane * KS;
      float s = 0.f;
      if (hd4) {
        const float4* q4 = reinterpret_cast<const float4*>(qv);
        const float4* k4 = reinterpret_cast<const float4*>(kr);
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int d = 0; d < hd / 4; d++) {
          const float4 a = q4[d], c = k4[d];
          s4[0] = fmaf(a.x, c.x, s4[0]);
          s4[1] = fmaf(a.y, c.y, s4[1]);
          s4[2] = fmaf(a.z, c.z, s4[2]);
          s4[3] = fmaf(a.w, c.w, s4[3]);
        }
        s = (s4[0] + s4[1]) + (s4[2] + s4[3]);
      } else {
#pragma unroll 8
        for (int d = 0; d < hd; d++) s += qv[d] * kr[d];
      }
      s *= head_scale[h];
      const int kp_ = key0 + lane;
      const bool valid = pooled ? kp_ < blocks_seen(qpos, window, pool)
                                : (kp_ <= qpos && (window <= 0 || kp_ + window > qpos));
      s = valid ? s : PAT_NEG;
      const float mn = fmaxf(mx[ri], warp_max(s));
      const float p = valid ? expf(s - mn) : 0.f;
      const float corr = expf(mx[ri] - mn);
      l[ri] = l[ri] * corr + warp_sum(p);
      mx[ri] = mn;
      p_s[warp * 32 + lane] = p;
      __syncwarp();
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < vd) {
          const float4* p4 = reinterpret_cast<const float4*>(p_s + warp * 32);
          const float4* v4 = reinterpret_cast<const float4*>(v_s + d * VS);
          float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int kk = 0; kk < 8; kk++) {
            const float4 pw = p4[kk], vv = v4[kk];
            a4[0] = fmaf(pw.x, vv.x, a4[0]);
            a4[1] = fmaf(pw.y, vv.y, a4[1]);
            a4[2] = fmaf(pw.z, vv.z, a4[2]);
            a4[3] = fmaf(pw.w, vv.w, a4[3]);
          }
          acc[ri][jj] = acc[ri][jj] * corr + ((a4[0] + a4[1]) + (a4[2] + a4[3]));
        }
      }
      __syncwarp();
    }
  }

  const int half = vd / 2;
#pragma unroll
  for (int ri = 0; ri < PAT_RPW; ri++) {
    const int r = warp + ri * PAT_WARPS;
    if (r >= R) break;
    const int i = r / HC, j = r % HC;
    if (i >= nrows || j >= nheads) continue;
    const int h = kvh * G + hc * HC + j;
    const size_t m = (size_t)q0 + row_lo + i;
    if (n_splits == 1) {
      const float inv = l[ri] > 0.f ? 1.0f / l[ri] : 0.f;
      float* ow = o_s + warp * vd;
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < vd) ow[d] = acc[ri][jj] * inv;
      }
      __syncwarp();
      const float fpos = (float)(pos0 + row_lo + i);
      for (int d = lane; d < vd; d += 32) {
        float val = ow[d];
        if (freq_v) {       // turned back by the query's position
          const int pr = d < half ? d : d - half;
          float sn, cs;
          sincosf(fpos * freq_v[pr], &sn, &cs);
          val = d < half ? ow[d] * cs + ow[d + half] * sn : ow[d] * cs - ow[d - half] * sn;
        }
        out[(m * nh + h) * vd + d] = from_f32<T>(val);
      }
      __syncwarp();
    } else {
      float* pp = part + ((m * nh + h) * n_splits + split) * (size_t)(vd + 2);
      if (lane == 0) { pp[0] = mx[ri]; pp[1] = l[ri]; }
#pragma unroll
      for (int jj = 0; jj < HDL; jj++) {
        const int d = lane + 32 * jj;
        if (d < vd) pp[2 + d] = acc[ri][jj];
      }
    }
  }
}

// Merge of the splits of one (row, head), then the turn back by the row's position.
template <typename T>
__global__ void __launch_bounds__(64)
attention_pooled_merge_kernel(T* __restrict__ out, const float* __restrict__ part, const float* __restrict__ freq_v,
                              const int* __restrict__ row_pos, int nh, int vd, int n_splits) {
  pdl_wait();
  const size_t m = blockIdx.x;
  const int h = blockIdx.y;
  const size_t step = vd + 2;
  const float* pp = part + ((m * nh + h) * n_splits) * step;
  const int half = vd / 2;
  const float fpos = (float)row_pos[m];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float M = PAT_NEG;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, pp[s * step]);
    float L = 0.f, a0 = 0.f, a1 = 0.f;
    for (int s = 0; s < n_splits; s++) {
      const float* r = pp + s * step;
      const float e = expf(r[0] - M);
      L += r[1] * e;
      a0 += r[2 + i] * e;
      a1 += r[2 + i + half] * e;
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    a0 *= inv;
    a1 *= inv;
    float o0 = a0, o1 = a1;
    if (freq_v) {
      float sn, cs;
      sincosf(fpos * freq_v[i], &sn, &cs);
      o0 = a0 * cs + a1 * sn;
      o1 = a1 * cs - a0 * sn;
    }
    out[(m * nh + h) * vd + i] = from_f32<T>(o0);
    out[(m * nh + h) * vd + i + half] = from_f32<T>(o1);
  }
}

template <typename T, typename CT, int HDL>
static int launch_attention_pooled(void* out, float* part, const void* q, const void* k_pool, const void* v_pool,
                                   const int* block_table, int bt_width, const void* pk_pool, const void* pv_pool,
                                   const int* pool_table, int pt_width, const int* seq_slot, const int* seq_pos0,
                                   const int* seq_qstart, const int* seq_qlen, const float* head_scale, const float* freq_v,
                                   int B, int nh, int nkv, int hd, int vd, int page_size, int window, int pool, int max_qlen,
                                   int n_splits, cudaStream_t st) {
  const int G = nh / nkv;
  const int HC = G < 8 ? G : 8;
  int QT = 32 / HC;
  if (QT > max_qlen) QT = max_qlen;
  const int R = QT * HC;
  const int n_hc = ceil_div(G, HC);
  const size_t smem = ((size_t)((R * hd + 3) & ~3) + 32 * (((hd + 3) & ~3) + 4) + 36 * vd + PAT_WARPS * 32 + PAT_WARPS * vd) * sizeof(float);
  auto kern = attention_pooled_kernel<T, CT, HDL>;
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return leb_fail("leb_attention_pooled: shared memory %zu: %s", smem, cudaGetErrorString(e));
    smem_set = smem;
  }
  dim3 grid(ceil_div(max_qlen, QT), nkv * n_hc, B * n_splits);
  LEB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "leb_attention_pooled: grid too large (%u, %u)", grid.y, grid.z);
  leb_launch(kern, grid, dim3(32 * PAT_WARPS), smem, st, (T*)out, part, (const T*)q, (const CT*)k_pool, (const CT*)v_pool,
             block_table, bt_width, (const CT*)pk_pool, (const CT*)pv_pool, pool_table, pt_width, seq_slot, seq_pos0,
             seq_qstart, seq_qlen, head_scale, freq_v, nh, nkv, hd, vd, page_size, window, pool, QT, HC, n_splits);
  LEB_CHECK_LAUNCH("leb_attention_pooled");
  return 0;
}

// q [M, nh*hd], out [M, nh*vd] in the activation type (the cache's type as well); pools as the cache lays
// them out; head_scale [nh] float; freq_v [vd/2] float or null (values not rotated); part: float scratch
// of M*nh*n_splits*(vd+2) numbers for n_splits > 1 (one row per sequence then); row_pos [M].
LEB_API int leb_attention_pooled(void* out, float* part, const void* q, const void* k_pool, const void* v_pool, int dtype,
                                 const int* block_table, int bt_width, const void* pk_pool, const void* pv_pool,
                                 const int* pool_table, int pt_width, const int* seq_slot, const int* seq_pos0,
                                 const int* seq_qstart, const int* seq_qlen, const int* row_pos, const float* head_scale,
                                 const float* freq_v, int M, int B, int nh, int nkv, int hd, int vd, int page_size, int window,
                                 int pool, int max_qlen, int n_splits, cudaStream_t st) {
  if (M <= 0 || B <= 0) return 0;
  LEB_REQUIRE(vd >= 2 && vd <= 256 && vd % 2 == 0, "leb_attention_pooled: value head size %d outside 2..256 or odd", vd);
  LEB_REQUIRE(hd >= 1 && hd <= 256, "leb_attention_pooled: head_dim %d outside 1..256", hd);
  LEB_REQUIRE(nkv > 0 && nh % nkv == 0, "leb_attention_pooled: %d heads do not divide into %d kv heads", nh, nkv);
  LEB_REQUIRE(page_size % 32 == 0, "leb_attention_pooled: page size %d is not a multiple of 32", page_size);
  LEB_REQUIRE(n_splits >= 1 && (n_splits == 1 || (max_qlen == 1 && part)), "leb_attention_pooled: splits need single-row sequences and scratch");
  LEB_REQUIRE(pool <= 0 || (pk_pool && pv_pool && pool_table), "leb_attention_pooled: pooled blocks need their pools");
  LebPlainLaunches plain(true);
  int rc;
#define LEB_PAT_ARGS out, part, q, k_pool, v_pool, block_table, bt_width, pk_pool, pv_pool, pool_table, pt_width, seq_slot, \
                     seq_pos0, seq_qstart, seq_qlen, head_scale, freq_v, B, nh, nkv, hd, vd, page_size, window, pool, max_qlen, n_splits, st
#define LEB_PAT(T, CT)                                                   \
  (vd <= 32    ? launch_attention_pooled<T, CT, 1>(LEB_PAT_ARGS)         \
   : vd <= 64  ? launch_attention_pooled<T, CT, 2>(LEB_PAT_ARGS)         \
   : vd <= 128 ? launch_attention_pooled<T, CT, 4>(LEB_PAT_ARGS)         \
               : launch_attention_pooled<T, CT, 8>(LEB_PAT_ARGS))
  if (dtype == LEB_F32) rc = LEB_PAT(float, float);
  else if (dtype == LEB_BF16) rc = LEB_PAT(bf16, bf16);
  else return leb_fail("leb_attention_pooled: unknown dtype %d", dtype);
#undef LEB_PAT
#undef LEB_PAT_ARGS
  if (rc) return rc;
  if (n_splits > 1) {
    const dim3 grid(M, nh);
    if (dtype == LEB_F32)
      leb_launch(attention_pooled_merge_kernel<float>, grid, dim3(64), 0, st, (float*)out, part, freq_v, row_pos, nh, vd, n_splits);
    else
      leb_launch(attention_pooled_merge_kernel<bf16>, grid, dim3(64), 0, st, (bf16*)out, part, freq_v, row_pos, nh, vd, n_splits);
    LEB_CHECK_LAUNCH("leb_attention_pooled merge");
  }
  return 0;
}
