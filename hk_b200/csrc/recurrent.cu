// Recurrent mixers: scans over the rows of every request of a step, with the state of a request kept in
// float32 in its state slot between steps.
//
// A step's batch is described by a segment table int32 [n_seg, 3] = (state slot, first row, rows): the rows
// of a request are consecutive and in increasing position.  Every scan walks a segment's rows in order, one
// token after the other, whatever the cut of the prompt was, so the state after a token (and every sum's
// order) depends on the tokens before it alone: never on the portion sizes, the batch or the slot.
//
//   * generalised delta rule (per head a matrix state S [dk, dv]):
//         S_t = diag(d_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,   o_t = S_t^T r_t
//     with the decay d_t = exp(-decay_scale * sigmoid(wl_t + w0)), the removal rate a_t = sigmoid(al_t + a0) and
//     the unit key u_t = k_t / sqrt(sum(k_t^2) + key_eps).  The columns of S (one per value channel) never mix:
//     a thread group owns one column, its dk entries spread over L lanes in registers, so a token costs two
//     dot products over dk and no synchronisation.  What a token brings (d, a*u, u, k, r, v) is prepared for all
//     tokens at once by a kernel of its own and reaches the scan in chunks through shared memory.
//   * gate of the delta rule's output: each head's o over its root mean square, times a weight, times
//     sigmoid(g), narrowed to the compute type for the output projection.
//   * minGRU (one scalar state per channel): S_t = (1 - z_t) S_(t-1) + z_t c_t with z_t = sigmoid(zl_t + bz),
//     c_t = x + 1/2 for x >= 0 and sigmoid(x) below, x = xl_t + bx; output S_t * silu(g_t).
//
// All arithmetic is float32; the projections that feed the scans arrive as float32.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------ generalised delta rule: what a token brings
// One warp per (token, head) writes the record that the scan reads: five vectors of P = L * RPT floats (d, a*u, u, k, r;
// P >= dk, the rest zero) and the dv values.  Inside a vector, entry i sits at (i % L) * RPT + i / L: lane `sub` of a
// column's L lanes owns the entries i = sub, sub + L, ... and finds them side by side.  Everything that does not depend
// on the state is computed here, for all tokens at once.
__global__ void delta_rule_prep_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                                       const float* __restrict__ al, long long ld, const float* __restrict__ wl, long long ldw,
                                       const float* __restrict__ a_bias, const float* __restrict__ w_bias, float* __restrict__ rec,
                                       long long items, int H, int dk, int dv, int L, int RPT, float decay_scale, float key_eps) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const size_t row = (size_t)(item / H);
  const int h = (int)(item % H);
  const size_t hoff = (size_t)h * dk;
  const float* kp = k + row * ld + hoff;
  float ss = 0.f;
  for (int i = lane; i < dk; i += 32) {
    const float kv = kp[i];
    ss = fmaf(kv, kv, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss + key_eps);
  const int P = L * RPT;
  float* out = rec + (size_t)item * (5 * P + dv);
  for (int j = lane; j < P; j += 32) {
    const int i = (j % RPT) * L + j / RPT;       // the entry that sits at place j
    float d = 0.f, au = 0.f, u = 0.f, kv = 0.f, rv = 0.f;
    if (i < dk) {
      kv = kp[i];
      u = kv * inv;
      au = sigmoid_f(al[row * ld + hoff + i] + a_bias[hoff + i]) * u;
      d = expf(-decay_scale * sigmoid_f(wl[row * ldw + hoff + i] + w_bias[hoff + i]));
      rv = r[row * ld + hoff + i];
    }
    out[j] = d;
    out[P + j] = au;
    out[2 * P + j] = u;
    out[3 * P + j] = kv;
    out[4 * P + j] = rv;
  }
  for (int c = lane; c < dv; c += 32) out[5 * P + c] = v[row * ld + (size_t)h * dv + c];
}

// ------------------------------------------------------------------ generalised delta rule: the scan
// A block owns `cols` columns of one head's state for one segment; a column's state entries are spread over L lanes, RPT
// per lane, in registers.  Records arrive in chunks of `chunk` tokens through a two-stage cp.async ring (the next chunk is
// on its way while this one is walked) and are read with 16-byte loads.  Per token the chain that the next token waits
// for is: u . S (four partial sums, then L lanes by shuffle), then one fused update per state entry; the output's dot
// product hangs off that chain.  How many lanes share a column is chosen by the launcher: one lane (no shuffle, the fewest
// instructions) when requests and heads alone give the SMs enough warps, more when a single request must be spread out.
__device__ __forceinline__ void dr_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int RPT, int L, int CPT>     // CPT: columns a lane group owns (they share every load of the token's vectors)
__global__ void __launch_bounds__(256)
delta_rule_scan_kernel(const float* __restrict__ rec, const int* __restrict__ segs, float* __restrict__ state,
                       float* __restrict__ out, int H, int dk, int dv, int cols, int chunk) {
  extern __shared__ __align__(16) float sm[];   // [2][chunk][5 P + dv]
  constexpr int P = L * RPT;
  const int R = 5 * P + dv;
  const int seg = blockIdx.x / H, h = blockIdx.x % H;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const int col0 = blockIdx.y * cols;
  const int tid = threadIdx.x;
  const int sub = tid % L, cidx = (tid / L) * CPT;           // first of this lane group's columns, within the block
  bool col_ok[CPT];
  int col[CPT];
  float S[CPT][RPT];
  float* sp = state + ((size_t)slot * H + h) * dk * dv;
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    col[c] = col0 + cidx + c;
    col_ok[c] = cidx + c < cols && col[c] < dv;
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
      const int i = sub + L * m;
      S[c][m] = (col_ok[c] && i < dk) ? sp[(size_t)i * dv + col[c]] : 0.f;
    }
  }
  const int pieces = R >> 2;                    // records are whole 16-byte pieces: P is a multiple of 8, dv of 4
  auto fetch = [&](int c) {                     // chunk c -> stage c & 1
    const int t0 = c * chunk, tc = min(chunk, count - t0);
    float* dst = sm + (size_t)(c & 1) * chunk * R;
    const float* src = rec + ((size_t)(row0 + t0) * H + h) * R;
    for (int t = 0; t < tc; ++t)
      for (int p = tid; p < pieces; p += blockDim.x) dr_cp_async16(dst + (size_t)t * R + 4 * p, src + (size_t)t * H * R + 4 * p);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const int nchunks = (count + chunk - 1) / chunk;
  float* op = out + (size_t)row0 * H * dv + (size_t)h * dv + col[0];
  const size_t ostep = (size_t)H * dv;
  const bool lead = sub == 0;
  const int mine = sub * RPT, vat = 5 * P + min(col[0], dv - CPT);
  fetch(0);
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) {
      fetch(c + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int tc = min(chunk, count - c * chunk);
    const float* buf = sm + (size_t)(c & 1) * chunk * R + mine;
    const float* vbuf = sm + (size_t)(c & 1) * chunk * R + vat;
#pragma unroll 2
    for (int t = 0; t < tc; ++t) {
      const float* tok = buf + (size_t)t * R;
      float du[CPT][2];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) du[cc][0] = du[cc][1] = 0.f;
#pragma unroll
      for (int q = 0; q < RPT / 4; ++q) {
        const float4 u = *reinterpret_cast<const float4*>(tok + 2 * P + 4 * q);
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          du[cc][0] = fmaf(u.y, S[cc][4 * q + 1], fmaf(u.x, S[cc][4 * q], du[cc][0]));
          du[cc][1] = fmaf(u.w, S[cc][4 * q + 3], fmaf(u.z, S[cc][4 * q + 2], du[cc][1]));
        }
      }
      float dus[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) dus[cc] = du[cc][0] + du[cc][1];
#pragma unroll
      for (int o = L >> 1; o > 0; o >>= 1)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) dus[cc] += __shfl_xor_sync(0xffffffffu, dus[cc], o);
      float v[CPT], acc[CPT][2];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        v[cc] = vbuf[(size_t)t * R + cc];
        acc[cc][0] = acc[cc][1] = 0.f;
      }
#pragma unroll
      for (int q = 0; q < RPT / 4; ++q) {
        const float4 d = *reinterpret_cast<const float4*>(tok + 4 * q);
        const float4 au = *reinterpret_cast<const float4*>(tok + P + 4 * q);
        const float4 k = *reinterpret_cast<const float4*>(tok + 3 * P + 4 * q);
        const float4 r = *reinterpret_cast<const float4*>(tok + 4 * P + 4 * q);
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          float* Sc = S[cc];
          Sc[4 * q] = fmaf(k.x, v[cc], fmaf(-au.x, dus[cc], d.x * Sc[4 * q]));
          Sc[4 * q + 1] = fmaf(k.y, v[cc], fmaf(-au.y, dus[cc], d.y * Sc[4 * q + 1]));
          Sc[4 * q + 2] = fmaf(k.z, v[cc], fmaf(-au.z, dus[cc], d.z * Sc[4 * q + 2]));
          Sc[4 * q + 3] = fmaf(k.w, v[cc], fmaf(-au.w, dus[cc], d.w * Sc[4 * q + 3]));
          acc[cc][0] = fmaf(r.y, Sc[4 * q + 1], fmaf(r.x, Sc[4 * q], acc[cc][0]));
          acc[cc][1] = fmaf(r.w, Sc[4 * q + 3], fmaf(r.z, Sc[4 * q + 2], acc[cc][1]));
        }
      }
      float o_[CPT];
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) o_[cc] = acc[cc][0] + acc[cc][1];
#pragma unroll
      for (int o = L >> 1; o > 0; o >>= 1)
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) o_[cc] += __shfl_xor_sync(0xffffffffu, o_[cc], o);
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc)
        if (lead && col_ok[cc]) op[(size_t)t * ostep + cc] = o_[cc];
    }
    op += (size_t)tc * ostep;
    __syncthreads();                            // the stage may be filled again
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
      const int i = sub + L * m;
      if (col_ok[c] && i < dk) sp[(size_t)i * dv + col[c]] = S[c][m];
    }
}

// The plain form of the scan for value sizes that are no multiple of 4 (records that are not whole 16-byte pieces):
// the same recurrence, the state in shared memory, records read with plain loads, one token at a time.
__global__ void delta_rule_scan_plain_kernel(const float* __restrict__ rec, const int* __restrict__ segs, float* __restrict__ state,
                                             float* __restrict__ out, int H, int dk, int dv, int L, int RPT, int cols) {
  extern __shared__ __align__(16) float sm[];   // [blockDim / L][P] the state columns; then one record
  const int P = L * RPT, R = 5 * P + dv;
  const int seg = blockIdx.x / H, h = blockIdx.x % H;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const int tid = threadIdx.x, sub = tid % L, cidx = tid / L, col = blockIdx.y * cols + cidx;
  const bool col_ok = cidx < cols && col < dv;
  float* Sc = sm + (size_t)cidx * P;             // this column's state, in the record's order of entries
  float* recs = sm + (size_t)(blockDim.x / L) * P;
  float* sp = state + ((size_t)slot * H + h) * dk * dv;
  for (int m = 0; m < RPT; ++m) {
    const int i = sub + L * m;
    Sc[sub * RPT + m] = (col_ok && i < dk) ? sp[(size_t)i * dv + col] : 0.f;
  }
  for (int t = 0; t < count; ++t) {
    __syncthreads();
    const float* src = rec + ((size_t)(row0 + t) * H + h) * R;
    for (int p = tid; p < R; p += blockDim.x) recs[p] = src[p];
    __syncthreads();
    const float* mine = recs + sub * RPT;
    float du0 = 0.f, du1 = 0.f;
    for (int m = 0; m < RPT; m += 2) {
      du0 = fmaf(mine[2 * P + m], Sc[sub * RPT + m], du0);
      if (m + 1 < RPT) du1 = fmaf(mine[2 * P + m + 1], Sc[sub * RPT + m + 1], du1);
    }
    float du = du0 + du1;
    for (int o = L >> 1; o > 0; o >>= 1) du += __shfl_xor_sync(0xffffffffu, du, o);
    const float vj = recs[5 * P + min(col, dv - 1)];
    float a0 = 0.f, a1 = 0.f;
    for (int m = 0; m < RPT; ++m) {
      const float sn = fmaf(mine[3 * P + m], vj, fmaf(-mine[P + m], du, mine[m] * Sc[sub * RPT + m]));
      Sc[sub * RPT + m] = sn;
      if (m & 1) a1 = fmaf(mine[4 * P + m], sn, a1); else a0 = fmaf(mine[4 * P + m], sn, a0);
    }
    float acc = a0 + a1;
    for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (col_ok && sub == 0) out[(size_t)(row0 + t) * H * dv + (size_t)h * dv + col] = acc;
  }
  for (int m = 0; m < RPT; ++m) {
    const int i = sub + L * m;
    if (col_ok && i < dk) sp[(size_t)i * dv + col] = Sc[sub * RPT + m];
  }
}

// How a column's dk state entries are laid over lanes: L lanes with RPT entries each (RPT in 8, 16, 32, 64; L * RPT >= dk
// with as little padding as there can be).  `spread` asks for at least that many lanes: more warps for a small batch.
static void dr_layout(int dk, int spread, int* L_out, int* rpt_out) {
  int L = 1;
  while (L < 32 && (dk + L - 1) / L > 64) L <<= 1;
  while (L < 32 && L < spread && (dk + 2 * L - 1) / (2 * L) >= 8) L <<= 1;
  int rpt = 8;
  while (rpt < 64 && rpt * L < dk) rpt <<= 1;
  *L_out = L;
  *rpt_out = rpt * L >= dk ? rpt : 0;           // 0: dk above 2,048
}

// The most scratch floats per (token, head) that `hk_delta_rule_scan` may need in `rec`, whatever layout it chooses.
HK_API int hk_delta_rule_record(int dk, int dv) {
  int most = 0;
  for (int spread = 1; spread <= 32; spread <<= 1) {
    int L, rpt;
    dr_layout(dk, spread, &L, &rpt);
    if (rpt && 5 * L * rpt + dv > most) most = 5 * L * rpt + dv;
  }
  return most;
}

template <int RPT, int CPT>
static int dr_launch(int L, dim3 grid, int threads, size_t smem, cudaStream_t s, const float* rec, const int* segs, float* state,
                     float* out, int H, int dk, int dv, int cols, int chunk) {
#define DR_LAUNCH(LL)                                                                                                       \
  do {                                                                                                                      \
    static HkSmemCache cache;                                                                                               \
    int e = hk_allow_smem(delta_rule_scan_kernel<RPT, LL, CPT>, smem, cache);                                               \
    if (e) return e;                                                                                                        \
    return hk_launch(delta_rule_scan_kernel<RPT, LL, CPT>, grid, dim3(threads), smem, s, rec, segs, state, out, H, dk, dv, cols, \
                     chunk);                                                                                                \
  } while (0)
  switch (L) {
    case 1: DR_LAUNCH(1);
    case 2: DR_LAUNCH(2);
    case 4: DR_LAUNCH(4);
    case 8: DR_LAUNCH(8);
    case 16: DR_LAUNCH(16);
    default: DR_LAUNCH(32);
  }
#undef DR_LAUNCH
}

// `rec`: scratch of n_rows * H * hk_delta_rule_record(dk, dv) floats (16-byte aligned) that the call fills and reads.
HK_API int hk_delta_rule_scan(const float* r, const float* k, const float* v, const float* al, long long ld, const float* wl,
                              long long ldw, const float* a_bias, const float* w_bias, const int* segs, int n_seg, int n_rows,
                              float* rec, float* state, float* out, int H, int dk, int dv, float decay_scale, float key_eps,
                              void* stream) {
  if (n_seg <= 0 || n_rows <= 0) return 0;
  if (H < 1 || dk < 1 || dv < 1 || dk > 2048 || ((uintptr_t)rec & 15)) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  // lanes per column: one where requests x heads x columns alone give every SM four warps or more, else as many as that takes
  const long long warps1 = ((long long)n_seg * H * dv + 31) / 32;
  int spread = 1;
  while (spread < 32 && warps1 * spread < 4 * 148) spread <<= 1;
  int L, rpt;
  dr_layout(dk, spread, &L, &rpt);
  if (!rpt) return HK_ERR_UNSUPPORTED;
  const int R = 5 * L * rpt + dv;
  {
    const long long items = (long long)n_rows * H;
    int e = hk_launch(delta_rule_prep_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, s, r, k, v, al, ld, wl, ldw, a_bias,
                      w_bias, rec, items, H, dk, dv, L, rpt, decay_scale, key_eps);
    if (e) return e;
  }
  if (dv & 3) {
    const int cols = max(1, min(dv, 128 / L));
    const int threads = ((cols * L + 31) / 32) * 32;      // whole warps: the lanes of a column meet by shuffle
    const size_t smem = (size_t)(threads * rpt + R) * sizeof(float);
    static HkSmemCache cache;
    int e = hk_allow_smem(delta_rule_scan_plain_kernel, smem, cache);
    if (e) return e;
    return hk_launch(delta_rule_scan_plain_kernel, dim3((unsigned)(n_seg * H), (unsigned)((dv + cols - 1) / cols)), dim3(threads), smem, s,
                     (const float*)rec, segs, state, out, H, dk, dv, L, rpt, cols);
  }
  // a block takes as many columns as 256 threads hold (they share the records that the ring brings), fewer while the
  // blocks do not yet fill the SMs twice: one request of 2,048 tokens at 32 heads of 64 runs 808 us with 8 columns a
  // block (256 blocks of 64 threads) against 1,096 with 32 and 839 with 4; below 4 every block fetches too much
  int cols = max(1, min(dv, 256 / L));
  while (cols > 8 && cols * L > 64 && (long long)n_seg * H * ((dv + cols - 1) / cols) < 2 * 148) cols >>= 1;
  // two columns a lane group where a lane holds 8 state entries a column (they share the loads of the token's vectors,
  // and their two chains of arithmetic hide each other's latency) and the block's columns are even
  // (one request of 2,048 tokens: 64 heads of 64, 512 blocks: 1.00 ms against 1.12; 32 heads, 256 blocks: 0.89 against 0.78,
  // so only where the blocks fill the SMs twice)
  const bool many = (long long)n_seg * H * ((dv + cols - 1) / cols) >= 2 * 148;
  const int cpt = (rpt == 8 && many && (cols & 1) == 0 && (dv & 1) == 0) ? 2 : 1;
  const int threads = ((cols / cpt * L + 31) / 32) * 32;
  int chunk = 16;
  while (chunk > 2 && (size_t)2 * chunk * R * sizeof(float) > 64 * 1024) chunk >>= 1;
  const size_t smem = (size_t)2 * chunk * R * sizeof(float);
  dim3 grid((unsigned)(n_seg * H), (unsigned)((dv + cols - 1) / cols));
  if (rpt == 8 && cpt == 2) return dr_launch<8, 2>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  if (rpt == 8) return dr_launch<8, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  if (rpt == 16) return dr_launch<16, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  if (rpt == 32) return dr_launch<32, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
  return dr_launch<64, 1>(L, grid, threads, smem, s, rec, segs, state, out, H, dk, dv, cols, chunk);
}

// ------------------------------------------------------------------ generalised delta rule: the output's gate
// One warp per (token, head): y = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g), narrowed to T.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ g, long long ldg,
                                      const float* __restrict__ weight, T* __restrict__ out, long long items, int H, int dv,
                                      float eps) {
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long long t = item / H;
  const int h = (int)(item % H);
  const float* src = o + (size_t)item * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) {
    const float a = src[i];
    ss = fmaf(a, a, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
  for (int i = lane; i < dv; i += 32) {
    const float gate = sigmoid_f(g[(size_t)t * ldg + (size_t)h * dv + i]);
    out[(size_t)item * dv + i] = from_f32<T>(src[i] * inv * weight[(size_t)h * dv + i] * gate);
  }
}

HK_API int hk_head_norm_gate(const float* o, const float* g, long long ldg, const float* weight, void* out, int out_dtype, int n,
                             int H, int dv, float eps, void* stream) {
  if (n <= 0) return 0;
  const long long items = (long long)n * H;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == HK_F32)
    return hk_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, s, o, g, ldg, weight, (float*)out, items, H, dv, eps);
  if (out_dtype == HK_BF16)
    return hk_launch(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, s, o, g, ldg, weight, (bf16*)out, items, H, dv, eps);
  return HK_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------ minGRU
// proj[n, 3W] = [z logits | candidate inputs | gate inputs].  A block owns 32 channels of a segment and walks it in
// chunks of MG_CHUNK tokens: all threads turn the chunk's inputs into a = 1 - z, b = z * c and silu(g) (in parallel,
// the next chunk's inputs already on their way in registers), one warp runs the recurrence S <- a S + b down the
// chunk, a channel per lane, and all threads write S * silu(g).
#define MG_CHUNK 64
#define MG_LANES 8      // token lanes: a thread takes every 8th token of a chunk in the parallel phases
#define MG_PER (MG_CHUNK / MG_LANES)

template <typename T>
__global__ void __launch_bounds__(32 * MG_LANES)
mingru_scan_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ z_bias,
                   const float* __restrict__ x_bias, const int* __restrict__ segs, float* __restrict__ state,
                   T* __restrict__ out, int W) {
  __shared__ float sa[MG_CHUNK][32], sb[MG_CHUNK][32], sg[MG_CHUNK][32];
  const int seg = blockIdx.x;
  const int ch = threadIdx.x & 31, tl = threadIdx.x >> 5;
  const int c = blockIdx.y * 32 + ch;
  const bool ok = c < W;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const float bz = (ok && z_bias) ? z_bias[c] : 0.f, bx = (ok && x_bias) ? x_bias[c] : 0.f;
  float S = (ok && tl == 0) ? state[(size_t)slot * W + c] : 0.f;
  if (count == 1) {                              // a decoded token: nothing to stage, one lane per channel does it all
    if (ok && tl == 0) {
      const float* p = proj + (size_t)row0 * ld + c;
      const float z = sigmoid_f(p[0] + bz);
      const float x = p[W] + bx;
      const float g = p[2 * (size_t)W];
      S = fmaf(1.0f - z, S, z * (x >= 0.f ? x + 0.5f : sigmoid_f(x)));
      out[(size_t)row0 * W + c] = from_f32<T>(S * (g * sigmoid_f(g)));
      state[(size_t)slot * W + c] = S;
    }
    return;
  }
  float zl[MG_PER], xl[MG_PER], gl[MG_PER];
  auto fetch = [&](int t0) {
#pragma unroll
    for (int j = 0; j < MG_PER; ++j) {
      const int t = t0 + tl + j * MG_LANES;
      const bool in = ok && t < count;
      const float* p = proj + (size_t)(row0 + (in ? t : 0)) * ld + (ok ? c : 0);
      zl[j] = in ? p[0] : 0.f;
      xl[j] = in ? p[W] : 0.f;
      gl[j] = in ? p[2 * (size_t)W] : 0.f;
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < count; t0 += MG_CHUNK) {
    const int tc = min(MG_CHUNK, count - t0);
#pragma unroll
    for (int j = 0; j < MG_PER; ++j) {
      const int t = tl + j * MG_LANES;
      const float z = sigmoid_f(zl[j] + bz);
      const float x = xl[j] + bx;
      const float cand = x >= 0.f ? x + 0.5f : sigmoid_f(x);
      sa[t][ch] = 1.0f - z;
      sb[t][ch] = z * cand;
      sg[t][ch] = gl[j] * sigmoid_f(gl[j]);
    }
    __syncthreads();
    if (t0 + MG_CHUNK < count) fetch(t0 + MG_CHUNK);      // in flight while the recurrence runs
    if (tl == 0) {
      for (int t = 0; t < tc; ++t) {
        S = fmaf(sa[t][ch], S, sb[t][ch]);
        sa[t][ch] = S;
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < MG_PER; ++j) {
      const int t = tl + j * MG_LANES;
      if (ok && t < tc) out[(size_t)(row0 + t0 + t) * W + c] = from_f32<T>(sa[t][ch] * sg[t][ch]);
    }
    __syncthreads();                                     // the chunk's arrays are free again
  }
  if (ok && tl == 0) state[(size_t)slot * W + c] = S;
}

HK_API int hk_mingru_scan(const float* proj, long long ld, const float* z_bias, const float* x_bias, const int* segs, int n_seg,
                          float* state, void* out, int out_dtype, int W, void* stream) {
  if (n_seg <= 0 || W <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((unsigned)n_seg, (unsigned)((W + 31) / 32));
  if (out_dtype == HK_F32)
    return hk_launch(mingru_scan_kernel<float>, grid, dim3(32 * MG_LANES), 0, s, proj, ld, z_bias, x_bias, segs, state, (float*)out, W);
  if (out_dtype == HK_BF16)
    return hk_launch(mingru_scan_kernel<bf16>, grid, dim3(32 * MG_LANES), 0, s, proj, ld, z_bias, x_bias, segs, state, (bf16*)out, W);
  return HK_ERR_UNSUPPORTED;
}
