// y[M,N] = x[M,K] W[N,K]^T for a handful of rows (decode steps: M <= 64), bfloat16.
//
// With so few rows the product is a stream over the weights: every byte of W is read
// once and the speed is that of the memory.  A block owns 16 rows of W (the M side of
// an m16n8k16 tensor-core tile: the weights are the A operand, the activations the B
// operand, "swap AB"), its 8 warps split K between them in interleaved chunks of 32
// elements, and the warps' partial sums are added in shared memory in a fixed order,
// so the result does not depend on timing.  Operands go from global memory straight
// into MMA fragments with 16-byte loads: a thread takes 8 consecutive k of a row and
// feeds them to two MMAs under a permutation of k that both operands share, which
// leaves the dot products unchanged and needs no shared-memory staging for W.
//
// Epilogues: bfloat16 or float rows; or SwiGLU, where the block also owns the 16 "up"
// rows that belong to its 16 "gate" rows and writes silu(gate) * up (reference
// model.py:514).
#include "common.cuh"
#include <cstdlib>

namespace {

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {  // weights: read once, do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_keep(const void* p) {    // activations: shared by every block
  return __ldg(reinterpret_cast<const uint4*>(p));
}

template <typename TO>
__device__ __forceinline__ void store_out(TO* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// NT: n-tiles of 8 activation rows (M <= 8 * NT).  SETS: 1, or 2 for SwiGLU (gate and up rows).
// WARPS: warps of a block that split K between them.  Fewer warps make blocks small enough that
// all of them are resident at once (no second, partly filled wave); more warps shorten the
// chain of memory round trips of a block when there are few blocks anyway.
// MINB: blocks per SM asked of the compiler.  With 8 rows (NT = 1) the kernel takes 70 registers, three blocks
// of 256 threads per SM; held to 64 it takes four, which is worth it only where it saves a wave (7,168 weight
// rows are 448 blocks: four blocks too many for three per SM on 148 SMs) and costs a little elsewhere.
// DEEP: twice as many chunks in flight per thread (half as many round trips to memory per block), at 2 blocks per SM:
// for products of so few blocks that no more than two fall to an SM anyway.
template <int NT, int SETS, typename TO, int WARPS, int MINB = 0, bool DEEP = false>
__global__ void __launch_bounds__(WARPS * 32, MINB) gemm_small_m_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W,
                                                               TO* __restrict__ out, int M, int N, int K, int lda, int ldw,
                                                               int ldc, int set_stride_rows) {
  constexpr int THREADS = WARPS * 32;
  constexpr int U = (NT <= 2 ? 4 : 2) * (DEEP ? 2 : 1);  // chunks in flight per thread
  __shared__ float red[WARPS][16][8 * NT + 1];
  const int n0 = blockIdx.x * 16;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n_chunks = (K + 31) / 32;

  float acc[SETS][NT][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.f;

  const __nv_bfloat16* wrow[SETS][2];
#pragma unroll
  for (int s = 0; s < SETS; ++s) {
    wrow[s][0] = W + (size_t)(n0 + s * set_stride_rows + g) * ldw;
    wrow[s][1] = W + (size_t)(n0 + s * set_stride_rows + g + 8) * ldw;
  }
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

  if constexpr (DEEP) {
    // Two halves of the chunks in flight take turns: while one is multiplied the other is on its way, so the
    // requests of a block never run dry between rounds (a round of this kernel is as long as the memory
    // needs for its bytes, and the pause between rounds was a fifth of the time of a long product).
    constexpr int H = U / 2;
    uint4 wa[H][SETS][2], wb[H][SETS][2], xa[H][NT], xb[H][NT];
    auto fetch = [&](uint4 (&wv)[H][SETS][2], uint4 (&xv)[H][NT], int c0) {
#pragma unroll
      for (int u = 0; u < H; ++u) {
        const int c = c0 + u * WARPS;
        const int k = c * 32 + t * 8;
        const bool ok = c < n_chunks && k < K;
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
          wv[u][s][0] = ok ? ld_stream(wrow[s][0] + k) : zero;
          wv[u][s][1] = ok ? ld_stream(wrow[s][1] + k) : zero;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const int m = j * 8 + g;
          xv[u][j] = (ok && m < M) ? ld_keep(x + (size_t)m * lda + k) : zero;
        }
      }
    };
    auto multiply = [&](const uint4 (&wv)[H][SETS][2], const uint4 (&xv)[H][NT]) {
#pragma unroll
      for (int u = 0; u < H; ++u) {
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
          const uint4 a = wv[u][s][0], b = wv[u][s][1];
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            mma_bf16(acc[s][j], a.x, b.x, a.y, b.y, xv[u][j].x, xv[u][j].y);
            mma_bf16(acc[s][j], a.z, b.z, a.w, b.w, xv[u][j].z, xv[u][j].w);
          }
        }
      }
    };
    fetch(wa, xa, warp);
    for (int c0 = warp; c0 < n_chunks; c0 += 2 * H * WARPS) {
      fetch(wb, xb, c0 + H * WARPS);
      multiply(wa, xa);
      fetch(wa, xa, c0 + 2 * H * WARPS);
      multiply(wb, xb);
    }
  } else
  for (int c0 = warp; c0 < n_chunks; c0 += WARPS * U) {
    uint4 wv[U][SETS][2];
    uint4 xv[U][NT];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = c0 + u * WARPS;
      const int k = c * 32 + t * 8;
      const bool ok = c < n_chunks && k < K;
#pragma unroll
      for (int s = 0; s < SETS; ++s) {
        wv[u][s][0] = ok ? ld_stream(wrow[s][0] + k) : zero;
        wv[u][s][1] = ok ? ld_stream(wrow[s][1] + k) : zero;
      }
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int m = j * 8 + g;
        xv[u][j] = (ok && m < M) ? ld_keep(x + (size_t)m * lda + k) : zero;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int s = 0; s < SETS; ++s) {
        const uint4 a = wv[u][s][0], b = wv[u][s][1];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          mma_bf16(acc[s][j], a.x, b.x, a.y, b.y, xv[u][j].x, xv[u][j].y);
          mma_bf16(acc[s][j], a.z, b.z, a.w, b.w, xv[u][j].z, xv[u][j].w);
        }
      }
    }
  }
  // add the warps' partial sums in warp order, one set (gate, up) after the other
  constexpr int OUTS = (16 * 8 * NT + THREADS - 1) / THREADS;
  float v[SETS][OUTS];
#pragma unroll
  for (int s = 0; s < SETS; ++s) {
    if (s > 0) __syncthreads();
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      red[warp][g][j * 8 + 2 * t] = acc[s][j][0];
      red[warp][g][j * 8 + 2 * t + 1] = acc[s][j][1];
      red[warp][g + 8][j * 8 + 2 * t] = acc[s][j][2];
      red[warp][g + 8][j * 8 + 2 * t + 1] = acc[s][j][3];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < OUTS; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      float a = 0.f;
      if (idx < 16 * 8 * NT) {
        const int m = idx / 16, r = idx % 16;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) a += red[w][r][m];
      }
      v[s][i] = a;
    }
  }
#pragma unroll
  for (int i = 0; i < OUTS; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    const int m = idx / 16, r = idx % 16;   // consecutive threads write consecutive columns of one output row
    if (idx >= 16 * 8 * NT || m >= M) continue;
    float y;
    if (SETS == 2) {
      const float gte = v[0][i];
      y = gte / (1.f + expf(-gte)) * v[SETS - 1][i];
    } else {
      y = v[0][i];
    }
    store_out<TO>(out + (size_t)m * ldc + n0 + r, y);
  }
}

template <int NT, int SETS, typename TO>
void launch(const void* x, const void* W, void* out, int M, int N, int K, int lda, int ldw, int ldc, int n_out, int set_stride,
            cudaStream_t stream) {
  const int tiles = n_out / 16;
  // measured on B200 (148 SMs): with gate and up rows in one block, 4 warps let all 688 blocks of
  // Yi-6B be resident at once (36 us instead of 44); elsewhere 8 warps are best (4 and 16 are slower)
#define GO_W(W_)                                                                                                  \
  gemm_small_m_kernel<NT, SETS, TO, W_><<<tiles, W_ * 32, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)W, \
                                                                        (TO*)out, M, N, K, lda, ldw, ldc, set_stride)
  if constexpr (SETS == 2) {
    GO_W(4);
  } else if constexpr (NT == 1) {
    const int sms = dk_sm_count();
    const int waves3 = (tiles + 3 * sms - 1) / (3 * sms), waves4 = (tiles + 4 * sms - 1) / (4 * sms);
    // (measured in the decode step of the Yi-6B shape, batch 8: 3.265 -> 3.227 ms with the deep instance for the
    // products of 256 blocks; held to three blocks per SM the compiler no longer keeps the loads in flight and nothing is gained)
    static const bool deep_off = getenv("DELTA_B200_SMALL_M_NO_DEEP") != nullptr;
    if (!deep_off && tiles <= 2 * sms)
      gemm_small_m_kernel<NT, SETS, TO, 8, 2, true><<<tiles, 8 * 32, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)W, (TO*)out, M, N,
                                                                                K, lda, ldw, ldc, set_stride);
    else if (waves4 < waves3)
      gemm_small_m_kernel<NT, SETS, TO, 8, 4><<<tiles, 8 * 32, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)W, (TO*)out, M, N, K,
                                                                          lda, ldw, ldc, set_stride);
    else
      GO_W(8);
  } else {
    GO_W(8);
  }
#undef GO_W
}
}  // namespace

extern "C" int dk_gemm_small_m_supported(int M, int N, int K, int swiglu) {
  if (M < 1 || M > 64 || K < 8 || (K % 8) != 0) return 0;
  const int n_out = swiglu ? N / 2 : N;
  if (swiglu && (N % 2) != 0) return 0;
  return (n_out % 16) == 0 ? 1 : 0;
}

// out_dtype: DK_BF16 or DK_F32.  swiglu: W = [gate rows; up rows] (N = 2 * I rows), out is [M, I].
extern "C" int dk_gemm_small_m(const void* x, const void* W, void* out, int M, int N, int K, int lda, int ldw, int ldc,
                               int out_dtype, int swiglu, cudaStream_t stream) {
  DK_REQUIRE(dk_gemm_small_m_supported(M, N, K, swiglu),
             "gemm_small_m: sizes not taken (1 <= M <= 64, K a multiple of 8, output columns a multiple of 16): M=%d N=%d K=%d", M, N, K);
  DK_REQUIRE(lda >= K && ldw >= K && (lda % 8) == 0 && (ldw % 8) == 0, "gemm_small_m: leading sizes must be multiples of 8 and >= K");
  DK_REQUIRE(((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_small_m: operands must start on 16-byte boundaries");
  const int n_out = swiglu ? N / 2 : N;
  DK_REQUIRE(ldc >= n_out, "gemm_small_m: output leading size %d is below %d", ldc, n_out);
  DK_REQUIRE(!(swiglu && out_dtype != DK_BF16), "gemm_small_m: the SwiGLU epilogue writes bfloat16");
  const int nt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
#define GO(NT_)                                                                                                     \
  do {                                                                                                              \
    if (swiglu) launch<NT_, 2, __nv_bfloat16>(x, W, out, M, N, K, lda, ldw, ldc, n_out, n_out, stream);             \
    else if (out_dtype == DK_BF16) launch<NT_, 1, __nv_bfloat16>(x, W, out, M, N, K, lda, ldw, ldc, n_out, 0, stream); \
    else if (out_dtype == DK_F32) launch<NT_, 1, float>(x, W, out, M, N, K, lda, ldw, ldc, n_out, 0, stream);        \
    else DK_REQUIRE(false, "gemm_small_m: unknown output dtype %d", out_dtype);                                     \
  } while (0)
  if (nt == 1) GO(1);
  else if (nt == 2) GO(2);
  else if (nt == 4) GO(4);
  else GO(8);
#undef GO
  return dk_check_launch("gemm_small_m");
}
