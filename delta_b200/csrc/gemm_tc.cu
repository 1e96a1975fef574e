// y[M,N] = x[M,K] W[N,K]^T on the fifth-generation tensor cores, for decode steps (M up to
// 128 rows): the weights stream once through shared memory by TMA and never touch
// registers.  More rows (prompt portions) are taken in chunks of up to 256 by one block per
// (tile of W, chunk), as a measure of what the library's product is worth there.
//
// "Swap AB": a block owns 128 rows of W, which are the M side of a tcgen05.mma tile
// (A operand), and all M activation rows, padded to a multiple of 16, are its N side (B
// operand).  The accumulator D[128 x Mpad] lives in tensor memory (TMEM).
//
//   thread 0        producer: per stage up to four TMA boxes [128 x 64] of W (512 contiguous
//                   bytes of every weight row are asked for together, which the memory
//                   likes far better than 128) and as many boxes [Mpad x 64] of x, into a
//                   ring of shared-memory stages (128-byte swizzle), signalled by mbarrier
//                   transaction counts
//   thread 32       issues four tcgen05.mma (K = 16 each) per box from shared-memory
//                   descriptors; tcgen05.commit frees the stage and, at the end, signals
//                   the epilogue
//   all four warps  epilogue: tcgen05.ld their 32 lanes of D into shared memory, then store
//                   (bfloat16 or float, or silu(gate) * up), after adding the partial sums
//                   of the other blocks when K is split
//
// With split K the blocks of a cluster (2, 4 or 8 along K) each keep a float partial
// [Mpad x 128] in their own shared memory; after a cluster barrier block r of the cluster
// adds the partials of all blocks, in rank order, over distributed shared memory for its
// share of the rows and stores them.  The order is fixed, so results do not depend on timing.
//
// Every wait on an mbarrier is bounded: when it gives up the kernel records that in the
// error record, skips its stores, frees its tensor memory and returns.
#include "common.cuh"
#include "tcgen05_helpers.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {
constexpr int TILE_ROWS = 128;   // rows of W per block (UMMA M)
constexpr int KSTEP = 64;        // elements of K per TMA box: one 128-byte swizzle row
constexpr int KSUB_MAX = 4;      // boxes per stage
constexpr int TC_THREADS = 128;

struct TcArgs {
  void* out;         // [M, ldc] bfloat16 or float
  int* err;
  int M, N, K, ldc;
  int mpad;          // M rounded up to a multiple of 16: the N of the MMA
  int stages;
  int out_f32;
  int swiglu;        // rows of the tile: 64 gate rows then the 64 up rows that belong to them
  int n_up;          // first up row in W (= columns of the output) when swiglu
  int tmem_cols;
  int ksub;          // boxes of 64 elements of K per stage (4, or 2 or 1 when many rows leave less room)
  int chunks;        // groups of mpad rows of x: block (tile, chunk) makes rows [chunk * mpad, ...) of the tile's columns
};

__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                             const __grid_constant__ CUtensorMap map_x, const TcArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the ring of stages starts on a 1024-byte boundary (the swizzle pattern repeats every 1024 bytes)
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int a_bytes = TILE_ROWS * KSTEP * 2;          // one box of W
  const int b_bytes = a.mpad * KSTEP * 2;             // one box of x (a multiple of 2048)
  const int KSUB = a.ksub;
  const int stage_bytes = KSUB * (a_bytes + b_bytes);
  __shared__ __align__(8) unsigned long long bars[2 * 16 + 1];   // full[s], empty[s], tmem_full
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  cg::cluster_group cluster = cg::this_cluster();
  const int splits = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  // 128 rows of W (64 + 64 with the SwiGLU epilogue).  The chunks of one tile are neighbours in the grid, so that
  // a tile of W is fetched from memory once and then found in the L2 by the blocks of the other chunks.
  const int tile = blockIdx.x / a.chunks;
  const int m0 = (blockIdx.x % a.chunks) * a.mpad;    // first row of x and of the output of this block
  const int m_here = min(a.mpad, a.M - m0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rows_out = a.swiglu ? 64 : TILE_ROWS;    // output columns this tile makes
  const int n0 = tile * rows_out;

  const int k_steps_total = (a.K + KSTEP * KSUB - 1) / (KSTEP * KSUB);
  const int per = (k_steps_total + splits - 1) / splits;
  const int ks_begin = rank * per;
  const int ks_end = min(k_steps_total, ks_begin + per);
  const int n_steps = max(0, ks_end - ks_begin);
  const uint32_t full0 = s2u(&bars[0]), empty0 = s2u(&bars[16]), tfull = s2u(&bars[32]);
  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(tfull, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // one step of the ring: the boxes of W and of x for step i into stage i % stages
  auto request = [&](int i) {
    const int s = i % a.stages;
    const uint32_t dst0 = s2u(smem + (size_t)s * stage_bytes);
    mbar_expect_tx(full0 + 8 * s, (uint32_t)stage_bytes);
    for (int sub = 0; sub < KSUB; ++sub) {
      const int kc = ((ks_begin + i) * KSUB + sub) * KSTEP;     // past K the boxes are filled with zeros
      const uint32_t dst = dst0 + sub * a_bytes;
      if (a.swiglu) {
        tma_load_2d(dst, &map_w, kc, n0, full0 + 8 * s);                           // 64 gate rows
        tma_load_2d(dst + 64 * KSTEP * 2, &map_w, kc, a.n_up + n0, full0 + 8 * s);  // their 64 up rows
      } else {
        tma_load_2d(dst, &map_w, kc, n0, full0 + 8 * s);
      }
      tma_load_2d(dst0 + KSUB * a_bytes + sub * b_bytes, &map_x, kc, m0, full0 + 8 * s);   // rows past M are zeros
    }
  };
  // The first round of the ring needs nothing but the barriers this thread has just made: it is asked for
  // before the block meets, so that the memory is already at work while the tensor memory is handed out.
  const int ahead = min(n_steps, a.stages);
  if (tid == 0)
    for (int i = 0; i < ahead; ++i) request(i);
  if (warp == 1) {   // one warp allocates the tensor memory for the accumulator
    tmem_alloc(s2u(&tmem_base_slot), a.tmem_cols);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (tid == 0) {
    // producer
    for (int i = ahead; i < n_steps; ++i) {
      const int s = i % a.stages;
      if (!mbar_wait(empty0 + 8 * s, ((i / a.stages) - 1) & 1)) {
        failed = 1;
        break;
      }
      request(i);
    }
  } else if (tid == 32) {
    // MMA issuer
    const uint32_t idesc = instr_desc_bf16(TILE_ROWS, a.mpad);
    for (int i = 0; i < n_steps; ++i) {
      const int s = i % a.stages;
      if (!mbar_wait(full0 + 8 * s, (i / a.stages) & 1)) {
        failed = 1;
        break;
      }
      tc_fence_after();
      const uint32_t sa = s2u(smem + (size_t)s * stage_bytes);
      for (int sub = 0; sub < KSUB; ++sub) {
        const uint64_t da = smem_desc_k_major(sa + sub * a_bytes), db = smem_desc_k_major(sa + KSUB * a_bytes + sub * b_bytes);
#pragma unroll
        for (int k = 0; k < KSTEP / 16; ++k)
          umma(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || sub > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(empty0 + 8 * s);      // the stage is free once these MMAs have read it
    }
    umma_commit(tfull);                 // the accumulator is complete once everything issued is done
  }
  // epilogue: every warp reads its 32 lanes of D
  __syncwarp();
  bool good = true;
  if (n_steps > 0) good = mbar_wait(tfull, 0);
  tc_fence_after();
  __syncthreads();
  if (!good || failed) {
    if (tid == 0) dk_report(a.err, DK_DEV_TIMEOUT, blockIdx.x, rank, n_steps);
    good = false;
  }
  const int row = warp * 32 + lane;                  // row of D = row of the W tile
  float* part = reinterpret_cast<float*>(smem);       // [mpad][128] floats, reuses the stages
  // D -> shared memory, transposed so that a token's 128 outputs are contiguous
  for (int c0 = 0; c0 < a.mpad; c0 += 16) {
    float v[16];
    if (good && n_steps > 0) {
      tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) part[(size_t)(c0 + i) * TILE_ROWS + row] = v[i];
  }
  tc_fence_before();
  if (splits > 1) cluster.sync(); else __syncthreads();

  // Block r of the cluster finishes rows [r * share, (r + 1) * share) of the tile, eight output
  // columns of one token at a time: the partial sums of all blocks are asked for together (two
  // 16-byte loads from each block's shared memory), added in rank order, and stored with 16 bytes.
  const int share = rows_out / splits;          // a multiple of 8
  const int r_begin = rank * share;
  const int groups = share / 8;
  const float* parts[8];
#pragma unroll
  for (int b = 0; b < 8; ++b) parts[b] = (b < splits && splits > 1) ? cluster.map_shared_rank(part, b) : part;
  for (int item = tid; item < groups * m_here; item += TC_THREADS) {
    const int m = item / groups, r = r_begin + (item % groups) * 8;
    float4 g0[8], g1[8], u0[8], u1[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b < splits) {
        const float* src = parts[b] + (size_t)m * TILE_ROWS + r;
        g0[b] = *reinterpret_cast<const float4*>(src);
        g1[b] = *reinterpret_cast<const float4*>(src + 4);
        if (a.swiglu) {
          u0[b] = *reinterpret_cast<const float4*>(src + 64);
          u1[b] = *reinterpret_cast<const float4*>(src + 68);
        }
      }
    }
    float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, u[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (b < splits) {
        y[0] += g0[b].x; y[1] += g0[b].y; y[2] += g0[b].z; y[3] += g0[b].w;
        y[4] += g1[b].x; y[5] += g1[b].y; y[6] += g1[b].z; y[7] += g1[b].w;
        if (a.swiglu) {
          u[0] += u0[b].x; u[1] += u0[b].y; u[2] += u0[b].z; u[3] += u0[b].w;
          u[4] += u1[b].x; u[5] += u1[b].y; u[6] += u1[b].z; u[7] += u1[b].w;
        }
      }
    }
    const int n = n0 + r;
    if (good && n < (a.swiglu ? a.n_up : a.N)) {     // N and the first up row are multiples of 8: a group is in or out as a whole
      if (a.swiglu) {
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = y[i] / (1.f + expf(-y[i])) * u[i];
      }
      if (a.out_f32) {
        float* dst = (float*)a.out + (size_t)(m0 + m) * a.ldc + n;
        *reinterpret_cast<float4*>(dst) = make_float4(y[0], y[1], y[2], y[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(y[4], y[5], y[6], y[7]);
      } else {
        uint4 st;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(y[0], y[1]), p1 = __floats2bfloat162_rn(y[2], y[3]),
                       p2 = __floats2bfloat162_rn(y[4], y[5]), p3 = __floats2bfloat162_rn(y[6], y[7]);
        st.x = *reinterpret_cast<uint32_t*>(&p0);
        st.y = *reinterpret_cast<uint32_t*>(&p1);
        st.z = *reinterpret_cast<uint32_t*>(&p2);
        st.w = *reinterpret_cast<uint32_t*>(&p3);
        *reinterpret_cast<uint4*>((__nv_bfloat16*)a.out + (size_t)(m0 + m) * a.ldc + n) = st;
      }
    }
  }
  if (splits > 1) cluster.sync(); else __syncthreads();   // nobody leaves while its memory is still read
  if (warp == 1) {
    tmem_dealloc(tmem_base, a.tmem_cols);
  }
}

bool make_map(CUtensorMap* m, const void* base, int rows, int K, int ld, int box_rows) {
  return make_tensor_map_bf16(m, base, rows, K, ld, box_rows);
}
}  // namespace

extern "C" int dk_gemm_tc_supported(int M, int N, int K, int swiglu) {
  if (M < 1 || M > 128 || K < 64 || (K % 8) != 0) return 0;
  if (swiglu) {
    if ((N % 2) != 0 || ((N / 2) % 64) != 0) return 0;
  } else if ((N % 8) != 0) {
    return 0;
  }
  return 1;
}

// More than 128 rows (prompt portions): the same kernel with the rows of x in chunks of up to 256, one block per
// (tile of W, chunk); K is not split and a block has the SM to itself.
extern "C" int dk_gemm_tc_many_rows_supported(int M, int N, int K, int swiglu) {
  if (M <= 128 || M > (1 << 20)) return 0;
  return dk_gemm_tc_supported(128, N, K, swiglu);
}

// splits: blocks that share K as one cluster (1, 2, 4 or 8).  out_dtype DK_BF16 or DK_F32.
// per_sm: 1, or 2 to size the ring of stages so that two blocks share an SM's shared memory (stages of half the
// length): with more tiles than SMs but no more than twice as many (11,008 SwiGLU columns are 172 tiles), all
// blocks then run at once instead of a full wave and a short one.
extern "C" int dk_gemm_tc(const void* x, const void* W, void* out, int M, int N, int K, int lda, int ldw, int ldc,
                          int out_dtype, int swiglu, int splits, int per_sm, int* err, cudaStream_t stream) {
  DK_REQUIRE(per_sm == 1 || per_sm == 2, "gemm_tc: per_sm must be 1 or 2, got %d", per_sm);
  const bool many = M > 128;
  DK_REQUIRE(many ? dk_gemm_tc_many_rows_supported(M, N, K, swiglu) : dk_gemm_tc_supported(M, N, K, swiglu),
             "gemm_tc: sizes not taken: M=%d N=%d K=%d swiglu=%d", M, N, K, swiglu);
  DK_REQUIRE(!many || (splits == 1 && per_sm == 1), "gemm_tc: more than 128 rows go with splits=1 and per_sm=1 (got %d, %d)", splits, per_sm);
  DK_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "gemm_tc: splits must be 1, 2, 4 or 8, got %d", splits);
  DK_REQUIRE((lda % 8) == 0 && (ldw % 8) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0,
             "gemm_tc: operands must start on 16-byte boundaries with leading sizes that are multiples of 8");
  DK_REQUIRE(out_dtype == DK_BF16 || out_dtype == DK_F32, "gemm_tc: unknown output dtype %d", out_dtype);
  DK_REQUIRE((ldc % 8) == 0 && ((uintptr_t)out % 16) == 0,
             "gemm_tc: the output must start on a 16-byte boundary with a leading size that is a multiple of 8");
  TcArgs a;
  a.out = out;
  a.err = err;
  a.M = M; a.N = N; a.K = K; a.ldc = ldc;
  a.mpad = M > 256 ? 256 : (M + 15) / 16 * 16;
  a.chunks = (M + a.mpad - 1) / a.mpad;
  a.out_f32 = out_dtype == DK_F32;
  a.swiglu = swiglu;
  a.n_up = swiglu ? N / 2 : 0;
  a.tmem_cols = a.mpad <= 32 ? 32 : (a.mpad <= 64 ? 64 : (a.mpad <= 128 ? 128 : 256));
  const int a_bytes = TILE_ROWS * KSTEP * 2;
  const int b_bytes = a.mpad * KSTEP * 2;
  a.ksub = per_sm == 2 ? 2 : (a.mpad <= 64 ? KSUB_MAX : (a.mpad <= 128 ? 2 : 1));
  const int stage_bytes = a.ksub * (a_bytes + b_bytes);
  const int part_bytes = a.mpad * TILE_ROWS * 4;
  int stages = ((224 * 1024) / per_sm - 2048) / stage_bytes;
  if (stages > 8) stages = 8;
  DK_REQUIRE(stages >= 2, "gemm_tc: M=%d leaves no room for two stages", M);
  a.stages = stages;
  size_t smem = (size_t)stages * stage_bytes;
  if (smem < (size_t)part_bytes) smem = part_bytes;
  smem += 1024;
  CUtensorMap map_w, map_x;
  DK_REQUIRE(make_map(&map_w, W, N, K, ldw, swiglu ? 64 : TILE_ROWS), "gemm_tc: cannot encode the tensor map of W");
  DK_REQUIRE(make_map(&map_x, x, M, K, lda, a.mpad), "gemm_tc: cannot encode the tensor map of x");
  static size_t configured_on[DK_MAX_DEVICES] = {0};
  size_t& configured = configured_on[dk_current_device()];
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      dk_set_error("gemm_tc: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return DK_ERR_LAUNCH;
    }
    configured = smem;
  }
  const int rows_out = swiglu ? 64 : TILE_ROWS;
  const int n_out = swiglu ? N / 2 : N;
  const int tiles = (n_out + rows_out - 1) / rows_out;
  cudaLaunchConfig_t cfg = {};
  DK_REQUIRE((long long)tiles * a.chunks < (1ll << 31), "gemm_tc: too many blocks");
  cfg.gridDim = dim3(tiles * a.chunks, splits, 1);
  cfg.blockDim = dim3(TC_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = splits;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel, map_w, map_x, a);
  if (e != cudaSuccess) {
    dk_set_error("gemm_tc: launch failed: %s", cudaGetErrorString(e));
    return DK_ERR_LAUNCH;
  }
  return dk_check_launch("gemm_tc");
}
