// Attention over a compressed cache for bf16 serving: H query heads over ONE shared key/value head whose key is the
// whole cache row of DK numbers (a latent and a rotated part) and whose value is the row's first DV numbers.  Rows
// this wide (hundreds of numbers) do not fit the flash kernels' register budget: a query tile cannot live in
// registers, nor can one warp hold a row's DV output sums.  Here
//
//   * a CTA takes one work item (a run of consecutive query tokens of a request and a key range; the same items as
//     the flash kernels', cut on the host) with all H heads: 64 rows = (token, head) pairs;
//   * the query tile lies in shared memory (64 x DK) and is read as mma A fragments with ldmatrix;
//   * keys come in tiles of 32 cache rows through a double-buffered cp.async ring, read once for all heads and once
//     for both uses: as K (all DK columns) and as V (the first DV columns);
//   * eight warps = four groups of 16 rows x two halves.  For the scores the two warps of a group split the tile's
//     keys (16 each, all DK columns); they exchange row maxima and the probabilities (bf16) through shared memory;
//     for the weighted values they split the DV columns (each half's sums stay in registers: DVW / 2 floats a
//     thread) and both read all 32 keys.  Scores and sums run on mma.sync.m16n8k16 with fp32 accumulation, the
//     softmax state (max, sum) is fp32.
//
// A row at position p sees keys [max(0, p - window + 1), p].  With key splitting a CTA writes an unnormalised
// partial (values, max, sum) and `latent_combine_kernel` merges a row's partials in split order.
// Limits: H <= 64, DK a multiple of 16 up to 576, DV a multiple of 16 up to min(DK, 512).
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr int ROWS = 64;     // (token, head) rows of a CTA
constexpr int TK = 32;       // keys of a tile
constexpr int PLD = TK + 8;  // padded row of the probability tile

struct Item {
  int q_row0;     // row of the first query token in the batch
  int n_tokens;   // query tokens of this item
  int slot;       // request slot (row of the block table)
  int pos0;       // position of the first query token
  int kv_lo;      // first key this item may read
  int kv_hi;      // one past the last key
  int part;       // index of the partial in scratch, or -1: write the output directly
  int pad;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// the two warps that share 16 rows meet here (barrier ids 1..4; 0 is __syncthreads)
__device__ __forceinline__ void pair_sync(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

size_t latent_smem(int DK) {
  const size_t LD = (size_t)DK + 8;
  return (ROWS * LD + 2 * TK * LD + ROWS * PLD) * sizeof(bf16) + 4 * ROWS * sizeof(float) + 2 * TK * sizeof(int);
}

// DVW: value columns per half (a warp's output sums: DVW / 2 floats a thread); DV <= 2 * DVW
template <int DVW>
__global__ void __launch_bounds__(256, 1)
latent_flash_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages, const int* __restrict__ block_table,
                    int table_stride, const Item* __restrict__ items, bf16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int H, int DK, int DV, int page_tokens, int window, float scale_log2) {
  const int LD = DK + 8;                 // padded row: an odd number of 16-byte chunks, no ldmatrix conflicts
  const int CPR = DK / 8;                // 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                 // [ROWS][LD]
  bf16* ks = qs + ROWS * LD;                                    // [2][TK][LD]
  bf16* ps = ks + 2 * TK * LD;                                  // [ROWS][PLD]
  float* mx = reinterpret_cast<float*>(ps + ROWS * PLD);        // [2][ROWS] row maxima of the two key halves
  float* ls = mx + 2 * ROWS;                                    // [2][ROWS] row sums of the two key halves
  int* tile_rows = reinterpret_cast<int*>(ls + 2 * ROWS);       // [2][TK]

  const Item it = items[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the two warps of a row group are neighbours, so they sit on different tensor units of the SM: a decode step, which
  // fills one or two row groups, still keeps two or four of the four units busy
  const int rg = warp >> 1, half = warp & 1;
  const int qr = lane >> 2, qt = lane & 3;
  const int mi = lane >> 3, r8 = lane & 7;
  const int* bt = block_table + (size_t)it.slot * table_stride;

  int row[2], pos[2], lo[2];
  bool valid[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    row[i] = rg * 16 + qr + 8 * i;
    const int tq = row[i] / H;
    valid[i] = tq < it.n_tokens;
    pos[i] = it.pos0 + (valid[i] ? tq : 0);
    lo[i] = window > 0 ? max(0, pos[i] - window + 1) : 0;
  }

  // the query tile: rows past the item's tokens are zero
  // (a warp copies whole rows, a lane every 32nd chunk of a row: no division in the copy loops)
  for (int r = warp; r < ROWS; r += 8) {
    const int tq = r / H;
    const bool ok = tq < it.n_tokens;
    const bf16* src = q + ((size_t)(it.q_row0 + (ok ? tq : 0)) * H + (r - tq * H)) * DK;
    for (int c = lane; c < CPR; c += 32) cp_async16(qs + r * LD + c * 8, src + c * 8, ok);
  }

  float o[DVW / 8][4];
#pragma unroll
  for (int n = 0; n < DVW / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};

  const int t_begin = it.kv_lo / TK;
  const int t_end = (it.kv_hi + TK - 1) / TK;
  const bool active = rg * 16 < it.n_tokens * H;      // whether any of this warp's 16 rows is a (token, head) of the item

  auto load_tile = [&](int t, int stage) {
    bf16* kd = ks + stage * TK * LD;
    int* pg = tile_rows + stage * TK;          // per key: its row in the [rows, DK] view of the pages, or -1
    if (threadIdx.x < TK) {
      const int j = t * TK + threadIdx.x;
      int row_of_key = -1;
      if (j >= it.kv_lo && j < it.kv_hi) {
        const int pi = j / page_tokens;
        const int page = bt[pi];
        if (page >= 0) row_of_key = page * page_tokens + (j - pi * page_tokens);
      }
      pg[threadIdx.x] = row_of_key;
    }
    __syncthreads();
#pragma unroll
    for (int r = warp; r < TK; r += 8) {
      const int row_of_key = pg[r];
      const bool ok = row_of_key >= 0;
      const bf16* src = pages + (ok ? (size_t)row_of_key * DK : 0);
      for (int c = lane; c < CPR; c += 32) cp_async16(kd + r * LD + c * 8, src + c * 8, ok);
    }
  };

  if (t_begin < t_end) load_tile(t_begin, 0);
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    const int stage = (t - t_begin) & 1;
    if (t + 1 < t_end) load_tile(t + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* kt = ks + stage * TK * LD;
    if (!active) {             // a decode step fills few of the 64 rows: the other row groups only help with the loads
      __syncthreads();
      continue;
    }

    // ---- scores: this warp's 16 rows against its 16 keys of the tile, over all DK columns.  Four K slices at a time:
    // their eight fragment loads go out before the eight products that use them, and every fourth slice adds onto the
    // same partial sums, so a product never waits for the one before it.
    float sp[4][2][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) sp[u][n][e] = 0.f;
    const bf16* qa = qs + (rg * 16 + r8 + (mi & 1) * 8) * LD + (mi >> 1) * 8;
    const bf16* kb = kt + (half * 16 + (mi >> 1) * 8 + r8) * LD + (mi & 1) * 8;
    const int ksteps = DK / 16;
    for (int kk0 = 0; kk0 < ksteps; kk0 += 4) {
      uint32_t a[4][4], b[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (kk0 + u < ksteps) {
          ldmatrix_x4(a[u], qa + (kk0 + u) * 16);
          ldmatrix_x4(b[u], kb + (kk0 + u) * 16);
        }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (kk0 + u < ksteps) {
          mma_bf16(sp[u][0], a[u], b[u][0], b[u][1]);
          mma_bf16(sp[u][1], a[u], b[u][2], b[u][3]);
        }
    }
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = (sp[0][n][e] + sp[1][n][e]) + (sp[2][n][e] + sp[3][n][e]);
    float mt[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = t * TK + half * 16 + n * 8 + 2 * qt + (e & 1);
        const bool ok = valid[i] && j >= lo[i] && j <= pos[i] && j >= it.kv_lo && j < it.kv_hi;
        s[n][e] = ok ? s[n][e] * scale_log2 : -CUDART_INF_F;
        mt[i] = fmaxf(mt[i], s[n][e]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 1));
      mt[i] = fmaxf(mt[i], __shfl_xor_sync(0xffffffffu, mt[i], 2));
      if (qt == 0) mx[half * ROWS + row[i]] = mt[i];
    }
    pair_sync(1 + rg);
    float msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float mn = fmaxf(m[i], fmaxf(mx[row[i]], mx[ROWS + row[i]]));
      msafe[i] = mn == -CUDART_INF_F ? 0.f : mn;
      const float corr = exp2f(m[i] - msafe[i]);       // m = -inf -> 0
      m[i] = mn;
      l[i] *= corr;
#pragma unroll
      for (int n = 0; n < DVW / 8; ++n) {
        o[n][2 * i] *= corr;
        o[n][2 * i + 1] *= corr;
      }
    }
    // ---- probabilities of this warp's keys, handed to its partner through shared memory
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = exp2f(s[n][e] - msafe[e >> 1]);
        l[e >> 1] += p[e];
      }
      const int col = half * 16 + n * 8 + 2 * qt;
      *reinterpret_cast<uint32_t*>(ps + row[0] * PLD + col) = pack_bf16(p[0], p[1]);
      *reinterpret_cast<uint32_t*>(ps + row[1] * PLD + col) = pack_bf16(p[2], p[3]);
    }
    pair_sync(1 + rg);
    // ---- weighted values: all 32 keys, this warp's half of the value columns
    const bf16* pa = ps + (rg * 16 + r8 + (mi & 1) * 8) * PLD + (mi >> 1) * 8;
#pragma unroll
    for (int kk = 0; kk < TK / 16; ++kk) {
      uint32_t pf[4];
      ldmatrix_x4(pf, pa + kk * 16);
      const bf16* vb = kt + (kk * 16 + (mi & 1) * 8 + r8) * LD + half * DVW + (mi >> 1) * 8;
#pragma unroll
      for (int dp0 = 0; dp0 < DVW / 16; dp0 += 4) {       // four column pairs at a time: loads first, then the products
        uint32_t b[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (half * DVW + (dp0 + u) * 16 < DV) ldmatrix_x4_trans(b[u], vb + (dp0 + u) * 16);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (half * DVW + (dp0 + u) * 16 < DV) {
            mma_bf16(o[2 * (dp0 + u)], pf, b[u][0], b[u][1]);
            mma_bf16(o[2 * (dp0 + u) + 1], pf, b[u][2], b[u][3]);
          }
      }
    }
    __syncthreads();   // the stage, the maxima and the probability tile are free again
  }
  cp_async_wait<0>();

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    if (qt == 0) ls[half * ROWS + row[i]] = l[i];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float lt = ls[row[i]] + ls[ROWS + row[i]];
    if (it.part < 0) {
      if (!valid[i]) continue;
      const int tq = row[i] / H;
      bf16* op = out + ((size_t)(it.q_row0 + tq) * H + row[i] % H) * DV;
      const float inv = lt > 0.f ? 1.0f / lt : 0.f;
#pragma unroll
      for (int n = 0; n < DVW / 8; ++n) {
        const int d = half * DVW + n * 8 + 2 * qt;
        if (d < DV) *reinterpret_cast<uint32_t*>(op + d) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
      }
    } else {
      const size_t base = (size_t)it.part * ROWS + row[i];
      float* po = part_o + base * DV;
#pragma unroll
      for (int n = 0; n < DVW / 8; ++n) {
        const int d = half * DVW + n * 8 + 2 * qt;
        if (d < DV) *reinterpret_cast<float2*>(po + d) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      }
      if (half == 0 && qt == 0) *reinterpret_cast<float2*>(part_ml + base * 2) = make_float2(m[i], lt);
    }
  }
}

// Decode variant: the items of a step of single tokens fill 16 * MT of a tile's rows (one token, H <= 16 * MT heads), so
// the work of a key tile is spread the other way: tiles of 64 cache rows, and for the scores each of the eight warps takes
// 8 keys against all rows; the row maxima and the probabilities go through shared memory (CTA-wide barriers); for the
// weighted values each warp takes an eighth of the value columns over all 64 keys.  Per key a warp then issues an eighth
// of the products that the prompt variant's busiest warp does, and no warp idles.
constexpr int DTK = 64;       // keys of a tile
constexpr int DPLD = DTK + 8;

size_t latent_decode_smem(int DK, int MT) {
  const size_t LD = (size_t)DK + 8;
  return (16 * MT * LD + 2 * DTK * LD + 16 * MT * DPLD) * sizeof(bf16) + (8 + 8) * 16 * MT * sizeof(float) + 2 * DTK * sizeof(int);
}

// MT: 16-row tiles (1: up to 16 heads, 2: up to 32); DVC: value columns per warp (DV <= 8 * DVC)
template <int MT, int DVC>
__global__ void __launch_bounds__(256, 1)
latent_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages, const int* __restrict__ block_table,
                     int table_stride, const Item* __restrict__ items, bf16* __restrict__ out, float* __restrict__ part_o,
                     float* __restrict__ part_ml, int H, int DK, int DV, int page_tokens, int window, float scale_log2) {
  constexpr int R = 16 * MT;
  const int LD = DK + 8;
  const int CPR = DK / 8;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                 // [R][LD]
  bf16* ks = qs + R * LD;                                       // [2][DTK][LD]
  bf16* ps = ks + 2 * DTK * LD;                                 // [R][DPLD]
  float* mx = reinterpret_cast<float*>(ps + R * DPLD);          // [8][R] row maxima of the eight key slices
  float* ls = mx + 8 * R;                                       // [8][R] row sums of the eight key slices
  int* tile_rows = reinterpret_cast<int*>(ls + 8 * R);          // [2][DTK]

  const Item it = items[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qr = lane >> 2, qt = lane & 3;
  const int mi = lane >> 3, r8 = lane & 7;
  const int* bt = block_table + (size_t)it.slot * table_stride;
  const int pos = it.pos0;                                      // one token
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;

  for (int r = warp; r < R; r += 8) {
    const bool ok = r < H;
    const bf16* src = q + ((size_t)it.q_row0 * H + (ok ? r : 0)) * DK;
    for (int c = lane; c < CPR; c += 32) cp_async16(qs + r * LD + c * 8, src + c * 8, ok);
  }

  float o[MT][DVC / 8][4];
  float m[MT][2], l[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int n = 0; n < DVC / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[mt][n][e] = 0.f;
    m[mt][0] = m[mt][1] = -CUDART_INF_F;
    l[mt][0] = l[mt][1] = 0.f;
  }

  const int t_begin = it.kv_lo / DTK;
  const int t_end = (it.kv_hi + DTK - 1) / DTK;

  auto load_tile = [&](int t, int stage) {
    bf16* kd = ks + stage * DTK * LD;
    int* pg = tile_rows + stage * DTK;
    if (threadIdx.x < DTK) {
      const int j = t * DTK + threadIdx.x;
      int row_of_key = -1;
      if (j >= it.kv_lo && j < it.kv_hi) {
        const int pi = j / page_tokens;
        const int page = bt[pi];
        if (page >= 0) row_of_key = page * page_tokens + (j - pi * page_tokens);
      }
      pg[threadIdx.x] = row_of_key;
    }
    __syncthreads();
#pragma unroll
    for (int r = warp; r < DTK; r += 8) {
      const int row_of_key = pg[r];
      const bool ok = row_of_key >= 0;
      const bf16* src = pages + (ok ? (size_t)row_of_key * DK : 0);
      for (int c = lane; c < CPR; c += 32) cp_async16(kd + r * LD + c * 8, src + c * 8, ok);
    }
  };

  if (t_begin < t_end) load_tile(t_begin, 0);
  cp_async_commit();
  for (int t = t_begin; t < t_end; ++t) {
    const int stage = (t - t_begin) & 1;
    if (t + 1 < t_end) load_tile(t + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* kt = ks + stage * DTK * LD;

    // ---- scores: all rows against this warp's 8 keys; two K slices of 16 columns per fragment load of the keys
    float sp[2][MT][4];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sp[u][mt][e] = 0.f;
    // x4 of the keys: matrices (k 0-7, k 8-15, k 16-23, k 24-31) of the warp's 8 keys -> b0, b1 of two K slices
    const bf16* kb = kt + (warp * 8 + r8) * LD + mi * 8;
    const int kpairs = DK / 32;                    // DK is a multiple of 16: a last single slice is handled below
    for (int kp = 0; kp < kpairs; ++kp) {
      uint32_t b[4];
      ldmatrix_x4(b, kb + kp * 32);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a0[4], a1[4];
        const bf16* qa = qs + (mt * 16 + r8 + (mi & 1) * 8) * LD + (mi >> 1) * 8 + kp * 32;
        ldmatrix_x4(a0, qa);
        ldmatrix_x4(a1, qa + 16);
        mma_bf16(sp[0][mt], a0, b[0], b[1]);
        mma_bf16(sp[1][mt], a1, b[2], b[3]);
      }
    }
    if (DK & 16) {                                 // the odd slice: its fragment load reads 16 columns past DK only as padding rows allow
      uint32_t b[4];
      const bf16* kl = kt + (warp * 8 + r8) * LD + (mi & 1) * 8 + kpairs * 32;     // matrices 2, 3 repeat 0, 1
      ldmatrix_x4(b, kl);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint32_t a0[4];
        ldmatrix_x4(a0, qs + (mt * 16 + r8 + (mi & 1) * 8) * LD + (mi >> 1) * 8 + kpairs * 32);
        mma_bf16(sp[0][mt], a0, b[0], b[1]);
      }
    }
    float s[MT][4];
    const int j0 = t * DTK + warp * 8 + 2 * qt;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float mt0 = -CUDART_INF_F, mt1 = -CUDART_INF_F;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + (e & 1);
        const bool ok = j >= lo && j <= pos && j >= it.kv_lo && j < it.kv_hi;
        s[mt][e] = ok ? (sp[0][mt][e] + sp[1][mt][e]) * scale_log2 : -CUDART_INF_F;
      }
      mt0 = fmaxf(s[mt][0], s[mt][1]);
      mt1 = fmaxf(s[mt][2], s[mt][3]);
      mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 1));
      mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, 2));
      mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 1));
      mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, 2));
      if (qt == 0) {
        mx[warp * R + mt * 16 + qr] = mt0;
        mx[warp * R + mt * 16 + qr + 8] = mt1;
      }
    }
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      float msafe[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = mt * 16 + qr + 8 * i;
        float mn = m[mt][i];
#pragma unroll
        for (int w = 0; w < 8; ++w) mn = fmaxf(mn, mx[w * R + r]);
        msafe[i] = mn == -CUDART_INF_F ? 0.f : mn;
        const float corr = exp2f(m[mt][i] - msafe[i]);
        m[mt][i] = mn;
        l[mt][i] *= corr;
#pragma unroll
        for (int n = 0; n < DVC / 8; ++n) {
          o[mt][n][2 * i] *= corr;
          o[mt][n][2 * i + 1] *= corr;
        }
      }
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = exp2f(s[mt][e] - msafe[e >> 1]);
        l[mt][e >> 1] += p[e];
      }
      const int col = warp * 8 + 2 * qt;
      *reinterpret_cast<uint32_t*>(ps + (mt * 16 + qr) * DPLD + col) = pack_bf16(p[0], p[1]);
      *reinterpret_cast<uint32_t*>(ps + (mt * 16 + qr + 8) * DPLD + col) = pack_bf16(p[2], p[3]);
    }
    __syncthreads();
    // ---- weighted values: all 64 keys, this warp's DVC value columns
#pragma unroll
    for (int kk = 0; kk < DTK / 16; ++kk) {
      uint32_t pf[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(pf[mt], ps + (mt * 16 + r8 + (mi & 1) * 8) * DPLD + (mi >> 1) * 8 + kk * 16);
      const bf16* vb = kt + (kk * 16 + (mi & 1) * 8 + r8) * LD + warp * DVC + (mi >> 1) * 8;
#pragma unroll
      for (int dp = 0; dp < DVC / 16; ++dp) {
        if (warp * DVC + dp * 16 < DV) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vb + dp * 16);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16(o[mt][2 * dp], pf[mt], b[0], b[1]);
            mma_bf16(o[mt][2 * dp + 1], pf[mt], b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();   // the stage, the maxima and the probability tile are free again
  }
  cp_async_wait<0>();

#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float v = l[mt][i];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if (qt == 0) ls[warp * R + mt * 16 + qr + 8 * i] = v;
    }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = mt * 16 + qr + 8 * i;
      if (r >= H) continue;
      float lt = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) lt += ls[w * R + r];
      if (it.part < 0) {
        bf16* op = out + ((size_t)it.q_row0 * H + r) * DV;
        const float inv = lt > 0.f ? 1.0f / lt : 0.f;
#pragma unroll
        for (int n = 0; n < DVC / 8; ++n) {
          const int d = warp * DVC + n * 8 + 2 * qt;
          if (d < DV) *reinterpret_cast<uint32_t*>(op + d) = pack_bf16(o[mt][n][2 * i] * inv, o[mt][n][2 * i + 1] * inv);
        }
      } else {
        const size_t base = (size_t)it.part * ROWS + r;
        float* po = part_o + base * DV;
#pragma unroll
        for (int n = 0; n < DVC / 8; ++n) {
          const int d = warp * DVC + n * 8 + 2 * qt;
          if (d < DV) *reinterpret_cast<float2*>(po + d) = make_float2(o[mt][n][2 * i], o[mt][n][2 * i + 1]);
        }
        if (warp == 0 && qt == 0) *reinterpret_cast<float2*>(part_ml + base * 2) = make_float2(m[mt][i], lt);
      }
    }
}

// Merges the partials of every (token, head) whose keys were split: partial s of token t sits at row
// (first[t] + s) * ROWS + row0[t] + head.  One warp per (token, head); the partials are added in split order.
__global__ void latent_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      const int* __restrict__ first, const int* __restrict__ count,
                                      const int* __restrict__ row0, bf16* __restrict__ out, int n_tokens, int H, int DV) {
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= n_tokens * H) return;
  const int t = w / H, h = w % H;
  const int n = count[t];
  if (n <= 0) return;
  const size_t base0 = (size_t)first[t] * ROWS + row0[t] + h;
  float mm = -CUDART_INF_F;
  for (int s = 0; s < n; ++s) mm = fmaxf(mm, part_ml[(base0 + (size_t)s * ROWS) * 2]);
  constexpr int PER = 16;      // DV <= 512
  float acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  float lsum = 0.f;
  for (int s = 0; s < n; ++s) {
    const size_t b = base0 + (size_t)s * ROWS;
    const float2 ml = *reinterpret_cast<const float2*>(part_ml + b * 2);
    const float f = ml.x == -CUDART_INF_F ? 0.f : exp2f(ml.x - mm);
    lsum += ml.y * f;
    const float* po = part_o + b * DV;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + 32 * i;
      if (d < DV) acc[i] = fmaf(po[d], f, acc[i]);
    }
  }
  const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
  bf16* op = out + ((size_t)t * H + h) * DV;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = lane + 32 * i;
    if (d < DV) op[d] = __float2bfloat16_rn(acc[i] * inv);
  }
}

template <int DVW>
int launch_latent(const void* q, const void* pages, const int* bt, int stride, const void* items, int n_items, void* out,
                  float* part_o, float* part_ml, int H, int DK, int DV, int pt, int window, float scale_log2, cudaStream_t s) {
  const size_t smem = latent_smem(DK);
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(latent_flash_kernel<DVW>, smem, allowed)) return e;
  latent_flash_kernel<DVW><<<(unsigned)n_items, 256, smem, s>>>((const bf16*)q, (const bf16*)pages, bt, stride, (const Item*)items,
                                                                (bf16*)out, part_o, part_ml, H, DK, DV, pt, window, scale_log2);
  return hk_launch_status();
}

template <int MT, int DVC>
int launch_latent_decode(const void* q, const void* pages, const int* bt, int stride, const void* items, int n_items, void* out,
                         float* part_o, float* part_ml, int H, int DK, int DV, int pt, int window, float scale_log2, cudaStream_t s) {
  const size_t smem = latent_decode_smem(DK, MT);
  static HkSmemCache allowed = {};
  if (int e = hk_allow_smem(latent_decode_kernel<MT, DVC>, smem, allowed)) return e;
  latent_decode_kernel<MT, DVC><<<(unsigned)n_items, 256, smem, s>>>((const bf16*)q, (const bf16*)pages, bt, stride, (const Item*)items,
                                                                     (bf16*)out, part_o, part_ml, H, DK, DV, pt, window, scale_log2);
  return hk_launch_status();
}

}  // namespace

// q bf16 [n, H, DK]; pages bf16 [pages, 1, page_tokens, DK]; out bf16 [n, H, DV]; items as for the flash kernels, an item
// holding at most 64 / H query tokens; part_o [parts, 64, DV] and part_ml [parts, 64, 2] are fp32 scratch for items
// with part >= 0; scale_log2 = scale * log2(e).  single_tokens = 1 says that every item holds ONE token (a decode
// step): with up to 32 heads the variant that spreads a tile's keys over all warps takes it.
HK_API int hk_attention_latent(const void* q, const void* pages, const int* block_table, int table_stride, const void* items,
                               int n_items, void* out, float* part_o, float* part_ml, int H, int DK, int DV, int page_tokens,
                               int window, float scale_log2, int single_tokens, void* stream) {
  if (n_items <= 0) return 0;
  if (H < 1 || H > ROWS || DK < 16 || DK > 576 || (DK & 15) || DV < 16 || DV > DK || DV > 512 || (DV & 15) || page_tokens < 1)
    return HK_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)pages | (uintptr_t)out) & 15) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (single_tokens && H <= 32) {
#define HK_ARGS q, pages, block_table, table_stride, items, n_items, out, part_o, part_ml, H, DK, DV, page_tokens, window, scale_log2, s
    if (H <= 16) {
      if (DV <= 128) return launch_latent_decode<1, 16>(HK_ARGS);
      if (DV <= 256) return launch_latent_decode<1, 32>(HK_ARGS);
      return launch_latent_decode<1, 64>(HK_ARGS);
    }
    if (DV <= 128) return launch_latent_decode<2, 16>(HK_ARGS);
    if (DV <= 256) return launch_latent_decode<2, 32>(HK_ARGS);
    return launch_latent_decode<2, 64>(HK_ARGS);
#undef HK_ARGS
  }
  if (DV <= 128)
    return launch_latent<64>(q, pages, block_table, table_stride, items, n_items, out, part_o, part_ml, H, DK, DV, page_tokens, window, scale_log2, s);
  if (DV <= 256)
    return launch_latent<128>(q, pages, block_table, table_stride, items, n_items, out, part_o, part_ml, H, DK, DV, page_tokens, window, scale_log2, s);
  return launch_latent<256>(q, pages, block_table, table_stride, items, n_items, out, part_o, part_ml, H, DK, DV, page_tokens, window, scale_log2, s);
}

HK_API int hk_attention_latent_combine(const float* part_o, const float* part_ml, const int* first, const int* count,
                                       const int* row0, void* out, int n_tokens, int H, int DV, void* stream) {
  if (n_tokens <= 0) return 0;
  if (DV > 512) return HK_ERR_UNSUPPORTED;
  const int warps = 4;
  const unsigned grid = (unsigned)(((long long)n_tokens * H + warps - 1) / warps);
  return hk_launch(latent_combine_kernel, dim3(grid), dim3(warps * 32), 0, (cudaStream_t)stream, part_o, part_ml, first, count, row0,
                   (bf16*)out, n_tokens, H, DV);
}

HK_API int hk_attention_latent_rows() { return ROWS; }
