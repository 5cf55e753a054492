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
//     dot products over dk and no synchronisation.  What a token brings (d, a*u, u, k, r, v) is prepared for a
//     chunk of tokens at a time in shared memory.
//   * gate of the delta rule's output: each head's o over its root mean square, times a weight, times
//     sigmoid(g), narrowed to the compute type for the output projection.
//   * minGRU (one scalar state per channel): S_t = (1 - z_t) S_(t-1) + z_t c_t with z_t = sigmoid(zl_t + bz),
//     c_t = x + 1/2 for x >= 0 and sigmoid(x) below, x = xl_t + bx; output S_t * silu(g_t).
//
// All arithmetic is float32; the projections that feed the scans arrive as float32.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ------------------------------------------------------------------ generalised delta rule: the scan
#define DR_MAX_RPT 32   // state rows a thread holds at most: dk <= 32 * L, L <= 32

template <int RPT>
__global__ void delta_rule_scan_kernel(const float* __restrict__ r, const float* __restrict__ k, const float* __restrict__ v,
                                       const float* __restrict__ al, long long ld, const float* __restrict__ wl, long long ldw,
                                       const float* __restrict__ a_bias, const float* __restrict__ w_bias,
                                       const int* __restrict__ segs, float* __restrict__ state, float* __restrict__ out,
                                       int H, int dk, int dv, int L, int cols, int chunk, float decay_scale, float key_eps) {
  extern __shared__ float sm[];
  float* s_dec = sm;                          // [chunk][dk]
  float* s_au = s_dec + (size_t)chunk * dk;
  float* s_u = s_au + (size_t)chunk * dk;
  float* s_k = s_u + (size_t)chunk * dk;
  float* s_r = s_k + (size_t)chunk * dk;
  float* s_v = s_r + (size_t)chunk * dk;      // [chunk][cols]
  const int seg = blockIdx.x / H, h = blockIdx.x % H;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const int col0 = blockIdx.y * cols;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  const int sub = tid % L, col = col0 + tid / L;
  const bool col_ok = tid / L < cols && col < dv;
  float S[RPT];
  float* sp = state + ((size_t)slot * H + h) * dk * dv;
#pragma unroll
  for (int m = 0; m < RPT; ++m) {
    const int i = sub + L * m;
    S[m] = (col_ok && i < dk) ? sp[(size_t)i * dv + col] : 0.f;
  }
  const size_t hoff = (size_t)h * dk;
  for (int t0 = 0; t0 < count; t0 += chunk) {
    const int tc = min(chunk, count - t0);
    __syncthreads();                          // the chunk before is consumed
    for (int t = wid; t < tc; t += nw) {      // a warp prepares a token
      const size_t row = (size_t)(row0 + t0 + t);
      float ss = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float kv = k[row * ld + hoff + i];
        ss = fmaf(kv, kv, ss);
      }
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + key_eps);
      for (int i = lane; i < dk; i += 32) {
        const float kv = k[row * ld + hoff + i];
        const float u = kv * inv;
        const float a = sigmoid_f(al[row * ld + hoff + i] + a_bias[hoff + i]);
        const float d = expf(-decay_scale * sigmoid_f(wl[row * ldw + hoff + i] + w_bias[hoff + i]));
        s_dec[t * dk + i] = d;
        s_au[t * dk + i] = a * u;
        s_u[t * dk + i] = u;
        s_k[t * dk + i] = kv;
        s_r[t * dk + i] = r[row * ld + hoff + i];
      }
      for (int c = lane; c < cols; c += 32) s_v[t * cols + c] = col0 + c < dv ? v[row * ld + (size_t)h * dv + col0 + c] : 0.f;
    }
    __syncthreads();
    for (int t = 0; t < tc; ++t) {
      const float* pu = s_u + t * dk;
      float du = 0.f;
#pragma unroll
      for (int m = 0; m < RPT; ++m) {
        const int i = sub + L * m;
        if (i < dk) du = fmaf(pu[i], S[m], du);
      }
      for (int o = L >> 1; o > 0; o >>= 1) du += __shfl_xor_sync(0xffffffffu, du, o);
      const float vj = s_v[t * cols + min(tid / L, cols - 1)];
      float acc = 0.f;
#pragma unroll
      for (int m = 0; m < RPT; ++m) {
        const int i = sub + L * m;
        if (i < dk) {
          const float sn = fmaf(s_k[t * dk + i], vj, fmaf(-s_au[t * dk + i], du, s_dec[t * dk + i] * S[m]));
          S[m] = sn;
          acc = fmaf(s_r[t * dk + i], sn, acc);
        }
      }
      for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (col_ok && sub == 0) out[(size_t)(row0 + t0 + t) * H * dv + (size_t)h * dv + col] = acc;
    }
  }
#pragma unroll
  for (int m = 0; m < RPT; ++m) {
    const int i = sub + L * m;
    if (col_ok && i < dk) sp[(size_t)i * dv + col] = S[m];
  }
}

HK_API int hk_delta_rule_scan(const float* r, const float* k, const float* v, const float* al, long long ld, const float* wl,
                              long long ldw, const float* a_bias, const float* w_bias, const int* segs, int n_seg, float* state,
                              float* out, int H, int dk, int dv, float decay_scale, float key_eps, void* stream) {
  if (n_seg <= 0) return 0;
  if (H < 1 || dk < 1 || dv < 1 || dk > DR_MAX_RPT * 32) return HK_ERR_UNSUPPORTED;
  // lanes per column: the fewest that leave a thread at most 8 state rows while a block still has 32 threads or more
  int L = 1;
  while (L < 32 && (dk + L - 1) / L > 8) L <<= 1;
  while (L < 32 && dv * L < 64) L <<= 1;
  const int rpt = (dk + L - 1) / L;
  int cols = min(dv, 256 / L);
  if (cols < 1) cols = 1;
  int threads = ((cols * L + 31) / 32) * 32;
  const int chunk = dk > 64 ? 8 : 16;
  const size_t smem = (size_t)chunk * (5 * dk + cols) * sizeof(float);
  dim3 grid((unsigned)(n_seg * H), (unsigned)((dv + cols - 1) / cols));
  cudaStream_t s = (cudaStream_t)stream;
#define DR_LAUNCH(R)                                                                                                       \
  do {                                                                                                                     \
    static HkSmemCache cache;                                                                                              \
    int e = hk_allow_smem(delta_rule_scan_kernel<R>, smem, cache);                                                         \
    if (e) return e;                                                                                                       \
    return hk_launch(delta_rule_scan_kernel<R>, grid, dim3(threads), smem, s, r, k, v, al, ld, wl, ldw, a_bias, w_bias,     \
                     segs, state, out, H, dk, dv, L, cols, chunk, decay_scale, key_eps);                                   \
  } while (0)
  if (rpt <= 1) DR_LAUNCH(1);
  if (rpt <= 2) DR_LAUNCH(2);
  if (rpt <= 4) DR_LAUNCH(4);
  if (rpt <= 8) DR_LAUNCH(8);
  if (rpt <= 16) DR_LAUNCH(16);
  DR_LAUNCH(32);
#undef DR_LAUNCH
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
// proj[n, 3W] = [z logits | candidate inputs | gate inputs]; a thread owns a channel of a segment.
template <typename T>
__global__ void mingru_scan_kernel(const float* __restrict__ proj, long long ld, const float* __restrict__ z_bias,
                                   const float* __restrict__ x_bias, const int* __restrict__ segs, float* __restrict__ state,
                                   T* __restrict__ out, int W) {
  const int seg = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= W) return;
  const int slot = segs[seg * 3], row0 = segs[seg * 3 + 1], count = segs[seg * 3 + 2];
  const float bz = z_bias ? z_bias[c] : 0.f, bx = x_bias ? x_bias[c] : 0.f;
  float S = state[(size_t)slot * W + c];
  const float* p = proj + (size_t)row0 * ld + c;
  T* op = out + (size_t)row0 * W + c;
  float zl = p[0], xl = p[W], gl = p[2 * (size_t)W];
  for (int t = 0; t < count; ++t) {
    float zn = 0.f, xn = 0.f, gn = 0.f;
    if (t + 1 < count) {                       // the next token's inputs are asked for before this token's arithmetic
      const float* q = p + (size_t)(t + 1) * ld;
      zn = q[0];
      xn = q[W];
      gn = q[2 * (size_t)W];
    }
    const float z = sigmoid_f(zl + bz);
    const float x = xl + bx;
    const float cand = x >= 0.f ? x + 0.5f : sigmoid_f(x);
    S = (1.0f - z) * S + z * cand;
    op[(size_t)t * W] = from_f32<T>(S * (gl * sigmoid_f(gl)));
    zl = zn;
    xl = xn;
    gl = gn;
  }
  state[(size_t)slot * W + c] = S;
}

HK_API int hk_mingru_scan(const float* proj, long long ld, const float* z_bias, const float* x_bias, const int* segs, int n_seg,
                          float* state, void* out, int out_dtype, int W, void* stream) {
  if (n_seg <= 0 || W <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = W >= 128 ? 128 : 32 * ((W + 31) / 32);
  dim3 grid((unsigned)n_seg, (unsigned)((W + threads - 1) / threads));
  if (out_dtype == HK_F32)
    return hk_launch(mingru_scan_kernel<float>, grid, dim3(threads), 0, s, proj, ld, z_bias, x_bias, segs, state, (float*)out, W);
  if (out_dtype == HK_BF16)
    return hk_launch(mingru_scan_kernel<bf16>, grid, dim3(threads), 0, s, proj, ld, z_bias, x_bias, segs, state, (bf16*)out, W);
  return HK_ERR_UNSUPPORTED;
}
