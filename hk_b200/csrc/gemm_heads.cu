// One small bf16 product per head on the tensor cores: out[t, h, :N] = a[t, h, :K] * w[h]^T with w [heads][N][K].
// A mixer that keeps a compressed cache carries its queries into the latent space and its results out of it with
// such products (K and N of 128 to 512 per head, as many products as heads), too small each for the persistent
// tcgen05 kernel's tiles and too many for a launch apiece.
//
// A CTA of four warps computes 64 rows x 64 columns of one head (blockIdx.z): each warp 16 rows x 64 columns on
// mma.sync.m16n8k16 (bf16 in, fp32 accumulation in registers), operands through a two-stage cp.async ring of 64-wide
// K slices read with ldmatrix.  a's and out's rows and heads lie any number of elements apart (multiples of 8 for
// a, of 2 for out), so either may be a column slice of wider rows; out is bf16 or fp32.  Each output element sums
// k = 0..K-1 in one order whatever the batch, so a row's result does not depend on what else is in the step.
// With `gate` (fp32 logits [M, >= heads * N], row stride gate_ld, head h at column h * N) the result is multiplied by
// sigmoid(gate) in the epilogue: a mixer's output gate without a kernel of its own.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 64, LDS = BK + 8;

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
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename TO>
__device__ __forceinline__ void store2(TO* p, float x, float y);
template <>
__device__ __forceinline__ void store2<float>(float* p, float x, float y) { *reinterpret_cast<float2*>(p) = make_float2(x, y); }
template <>
__device__ __forceinline__ void store2<bf16>(bf16* p, float x, float y) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y); }

template <typename TO>
__global__ void __launch_bounds__(128)
gemm_heads_mma_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, TO* __restrict__ out, int M, int N, int K,
                      long long lda, long long a_head, long long ldo, long long o_head, const float* __restrict__ gate,
                      long long gate_ld) {
  __shared__ __align__(16) bf16 As[2][BM][LDS];
  __shared__ __align__(16) bf16 Ws[2][BN][LDS];
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qr = lane >> 2, qt = lane & 3, mi = lane >> 3, r8 = lane & 7;
  a += (size_t)h * a_head;
  w += (size_t)h * N * K;
  out += (size_t)h * o_head;
  float acc[BN / 8][4];
#pragma unroll
  for (int n = 0; n < BN / 8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;

  auto load = [&](int k0, int stage) {
    // 64 rows x 8 chunks of 8 for each operand: 512 chunks, four a thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 128;
      const int r = idx >> 3, c = (idx & 7) * 8;
      const bool ka = k0 + c < K;
      const bool oka = ka && m0 + r < M, okw = ka && n0 + r < N;
      cp_async16(&As[stage][r][c], a + (oka ? (size_t)(m0 + r) * lda + k0 + c : 0), oka);
      cp_async16(&Ws[stage][r][c], w + (okw ? (size_t)(n0 + r) * K + k0 + c : 0), okw);
    }
  };
  const int steps = (K + BK - 1) / BK;
  load(0, 0);
  cp_async_commit();
  for (int s = 0; s < steps; ++s) {
    const int stage = s & 1;
    if (s + 1 < steps) load((s + 1) * BK, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      uint32_t af[4];
      ldmatrix_x4(af, &As[stage][warp * 16 + r8 + (mi & 1) * 8][kk * 16 + (mi >> 1) * 8]);
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, &Ws[stage][np * 16 + (mi >> 1) * 8 + r8][kk * 16 + (mi & 1) * 8]);
        mma_bf16(acc[2 * np], af, b[0], b[1]);
        mma_bf16(acc[2 * np + 1], af, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int gm = m0 + warp * 16 + qr + 8 * i;
    if (gm >= M) continue;
    TO* o = out + (size_t)gm * ldo;
    const float* gr = gate ? gate + (size_t)gm * gate_ld + (size_t)h * N : nullptr;
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
      const int gn = n0 + n * 8 + 2 * qt;
      float x = acc[n][2 * i], y = acc[n][2 * i + 1];
      if (gr) {
        if (gn < N) x /= 1.0f + expf(-gr[gn]);
        if (gn + 1 < N) y /= 1.0f + expf(-gr[gn + 1]);
      }
      if (gn + 1 < N) store2<TO>(o + gn, x, y);
      else if (gn < N) o[gn] = from_f32<TO>(x);
    }
  }
}

}  // namespace

// Refuses (HK_ERR_UNSUPPORTED) what the 16-byte copies and paired stores cannot take: K, lda or a_head no multiple of
// 8, ldo or o_head odd, operands not 16-byte (out: 8-byte for fp32, 4-byte for bf16) aligned.
HK_API int hk_gemm_heads_mma(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K, int heads, long long lda,
                             long long a_head, long long ldo, long long o_head, const float* gate, long long gate_ld, void* stream) {
  if (M <= 0 || N <= 0 || heads <= 0) return 0;
  if (K <= 0 || (K & 7) || (lda & 7) || (a_head & 7) || (ldo & 1) || (o_head & 1)) return HK_ERR_UNSUPPORTED;
  if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & (out_dtype == HK_F32 ? 7 : 3))) return HK_ERR_UNSUPPORTED;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, heads);
  if (grid.y > 65535 || grid.z > 65535) return HK_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  if (out_dtype == HK_F32)
    return hk_launch_pdl(gemm_heads_mma_kernel<float>, grid, dim3(128), 0, s, (const bf16*)a, (const bf16*)w, (float*)out, M, N, K, lda,
                         a_head, ldo, o_head, gate, gate_ld);
  if (out_dtype == HK_BF16)
    return hk_launch_pdl(gemm_heads_mma_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)a, (const bf16*)w, (bf16*)out, M, N, K, lda,
                         a_head, ldo, o_head, gate, gate_ld);
  return HK_ERR_UNSUPPORTED;
}
