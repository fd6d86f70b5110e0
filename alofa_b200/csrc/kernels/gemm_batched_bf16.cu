// The batched product with strides of latent.cu on tensor cores, for bfloat16
// operands: out_b[m, n] = act(sum_k x_b[m, k] * w_b[n, k] + bias_b[n]) for
// every batch b (per-head products of latent attention), or, with tile_batch,
// one x and one out whose 64-row tiles each multiply by the weight of the
// batch the tile names (experts of a routed feed-forward, rows sorted by
// expert and padded to whole tiles).  64 x 64 output tile per CTA, 32-deep
// slices by cp.async into two shared-memory buffers, four warps of 32 x 32
// (mma.sync m16n8k16, fp32 sums), bias and activation on the fp32 sums.  The
// depth, the row strides and the batch strides are multiples of 8 elements and
// the operands start on 16-byte boundaries (the caller checks).
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 32, LD = TK + 8;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src)); }

template <typename TO>
__global__ void __launch_bounds__(128) gemm_batched_bf16_kernel(TO* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                const float* __restrict__ bias, const int* __restrict__ tile_batch, int M, int N,
                                                                int K, long long ldx, long long x_batch, long long ldw, long long w_batch,
                                                                long long ldo, long long out_batch, long long bias_batch, int act, int tile_rows) {
  __shared__ __align__(16) bf16 As[2][TM * LD];
  __shared__ __align__(16) bf16 Bs[2][TN * LD];
  pdl_begin();
  int b = blockIdx.z;
  if (tile_batch) {
    b = tile_batch[blockIdx.y * 64 / tile_rows];  // tile_rows is a multiple of this kernel's 64 rows
    if (b < 0) return;
  } else {
    x += (size_t)b * x_batch;
    out += (size_t)b * out_batch;
  }
  w += (size_t)b * w_batch;
  if (bias) bias += (size_t)b * bias_batch;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp & 1, wn = warp >> 1, g = lane >> 2, t = lane & 3;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  auto fetch = [&](int kt, int buf) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int e = tid + 128 * i;
      const int r = e >> 2, c = (e & 3) * 8;
      const int gk = kt * TK + c;
      bf16* da = &As[buf][r * LD + c];
      if (m0 + r < M && gk < K) cp16(smem_addr(da), x + (size_t)(m0 + r) * ldx + gk);
      else *reinterpret_cast<uint4*>(da) = make_uint4(0, 0, 0, 0);
      bf16* db = &Bs[buf][r * LD + c];
      if (n0 + r < N && gk < K) cp16(smem_addr(db), w + (size_t)(n0 + r) * ldw + gk);
      else *reinterpret_cast<uint4*>(db) = make_uint4(0, 0, 0, 0);
    }
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;
  const int slices = (K + TK - 1) / TK;
  fetch(0, 0);
  asm volatile("cp.async.commit_group;");
  for (int kt = 0; kt < slices; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < slices) fetch(kt + 1, buf ^ 1);
    asm volatile("cp.async.commit_group;");
    asm volatile("cp.async.wait_group 1;");
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < TK; ks += 16) {
      uint32_t a[2][4], bb[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) ldsm4(a[i], smem_addr(&As[buf][(wm * 32 + i * 16 + (lane & 15)) * LD + ks + (lane >> 4) * 8]));
#pragma unroll
      for (int j = 0; j < 2; ++j) ldsm4(bb[j], smem_addr(&Bs[buf][(wn * 32 + j * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks + ((lane >> 3) & 1) * 8]));
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          mma16816(acc[i][2 * j], a[i], bb[j][0], bb[j][1]);
          mma16816(acc[i][2 * j + 1], a[i], bb[j][2], bb[j][3]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int gm = m0 + wm * 32 + i * 16 + g + (k >> 1) * 8;
        const int gn = n0 + wn * 32 + j * 8 + 2 * t + (k & 1);
        if (gm < M && gn < N) out[(size_t)gm * ldo + gn] = from_f<TO>(activate(acc[i][j][k] + (bias ? bias[gn] : 0.f), act));
      }
}

}  // namespace

ALOFA_API int alofa_gemm_batched_bf16(void* out, const void* x, const void* w, const float* bias, const int* tile_batch, int batches, int M, int N, int K,
                                      long long ldx, long long x_batch, long long ldw, long long w_batch, long long ldo, long long out_batch,
                                      long long bias_batch, int act, int tile_rows, int out_bf16, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batches <= 0) return ALOFA_OK;
  if (tile_batch && (tile_rows <= 0 || tile_rows % TM)) return ALOFA_ERR_ARGUMENT;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || (x_batch & 7) || (w_batch & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ALOFA_ERR_ARGUMENT;
  if ((M + TM - 1) / TM > 65535 || batches > 65535) return ALOFA_ERR_ARGUMENT;
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, tile_batch ? 1 : batches);
  if (out_bf16)
    launch_dep(gemm_batched_bf16_kernel<bf16>, grid, dim3(128), 0, stream, (bf16*)out, (const bf16*)x, (const bf16*)w, bias, tile_batch, M, N, K, ldx, x_batch,
               ldw, w_batch, ldo, out_batch, bias_batch, act, tile_rows);
  else
    launch_dep(gemm_batched_bf16_kernel<float>, grid, dim3(128), 0, stream, (float*)out, (const bf16*)x, (const bf16*)w, bias, tile_batch, M, N, K, ldx,
               x_batch, ldw, w_batch, ldo, out_batch, bias_batch, act, tile_rows);
  return launch_status();
}
