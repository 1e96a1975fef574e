// y[M,N] = x[M,K] W[N,K]^T for decode steps with up to 128 rows, as one persistent kernel that
// streams W exactly once and keeps every SM streaming for the same time ("stream-K").
//
// The work is the sequence of (tile of 128 rows of W, step of K) pairs, tile after tile; a step is
// one shared-memory stage of 128 elements of K.  The sequence is cut into as many equal
// pieces as there are SMs and block b runs piece b in order.  So a block's TMA loads never drain
// between tiles (the producer keeps asking while the epilogue of the tile before is at work: two
// accumulators in tensor memory take turns), there is no partly filled last wave, and a product
// with few tiles still uses every SM.
//
// A piece that starts inside a tile ends that tile's sum for this block only: the block writes the
// float partial [rows x 128] to its slot of a workspace and raises its flag.  The block that holds
// the head of a tile (its steps from k = 0) owns the tile; the head comes at the end of its piece,
// while the other blocks ran their share of that tile first, so when the owner gets there the
// partials are there or about to be.  It adds them in block order (fixed: the result does not
// depend on timing) and stores the tile.  Flags carry the number of the launch, which the last
// block to finish counts up, so nothing has to be cleared and a stale flag is never taken.
//
//   warp 0   producer: per step two TMA boxes [128 x 64] of W and two [Mpad x 64] of x
//   warp 1   one thread issues tcgen05.mma (A = W tile from shared memory, B = x, D in TMEM)
//   warps 2-5 epilogue: TMEM -> shared memory (transposed), then 16-byte stores of bfloat16 or
//            float, or silu(gate) * up when the tile is 64 gate rows and their 64 up rows
//
// The blocks wait for one another, so the kernel is launched cooperatively (all blocks resident
// or the launch fails), and every wait, on an mbarrier or on a flag, gives up after two seconds:
// the kernel then records the fact, stores nothing more, frees its tensor memory and returns.
#include "common.cuh"
#include "tcgen05_helpers.cuh"

namespace {
constexpr int TILE_ROWS = 128;   // rows of W per tile (UMMA M)
constexpr int KSTEP = 64;        // elements of K per TMA box: one 128-byte swizzle row
constexpr int SK_THREADS = 192;  // producer warp, MMA warp, four epilogue warps
constexpr int EPI_THREADS = 128;
constexpr int MAX_STAGES = 8;

struct SkArgs {
  void* out;         // [M, ldc] bfloat16 or float
  int* err;
  float* ws;         // [blocks][mpad * 128] partial sums
  int* flags;        // {number of the last launch that ended, blocks done}, then per block: the launch whose partial is in its slot
  int M, N, K, ldc;
  int mpad;          // M rounded up to a multiple of 16: the N of the MMA
  int stages, ksub;  // ring of stages; boxes of 64 elements of K per stage
  int out_f32;
  int swiglu;        // rows of the tile: 64 gate rows then the 64 up rows that belong to them
  int n_up;          // first up row in W (= columns of the output) when swiglu
  int tmem_cols;
  int tiles, steps_per_tile;
  long long total;   // tiles * steps_per_tile
};

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

// false when the flag did not take the value within the limit
__device__ __forceinline__ bool flag_wait(const int* p, int want) {
  if (ld_acquire(p) == want) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t round = 0; round < SPIN_ROUNDS; ++round) {
    for (int i = 0; i < 64; ++i) {
      if (ld_acquire(p) == want) return true;
      __nanosleep(40);
    }
    if (global_timer_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
  return false;
}

__device__ __forceinline__ long long piece_begin(const SkArgs& a, int b, int blocks) { return a.total * b / blocks; }

// The order in which a block runs the L steps of its piece.  In sequence order the piece is: the
// rest of a tile that an earlier block began, whole tiles, the head of a tile that later blocks
// finish.  The head needs the other blocks' partial sums and the longest epilogue, so when there is
// a whole tile it is run before the last whole tile, whose main loop then hides that epilogue.
struct Piece {
  long long begin;
  int L;         // steps
  int T;         // steps of a tile
  int A;         // steps before the head in running order
  int head;      // steps of the head run out of order (0: sequence order)
};
__device__ __forceinline__ Piece make_piece(long long begin, long long end, int T) {
  Piece p;
  p.begin = begin;
  p.L = (int)(end - begin);
  p.T = T;
  const int k0 = (int)(begin % T);
  const int first_len = (T - k0) < p.L ? (T - k0) : p.L;
  const int rest = p.L - first_len;
  const int whole = rest / T, head = rest % T;
  const bool reorder = head > 0 && whole >= 1;
  p.head = reorder ? head : 0;
  p.A = reorder ? first_len + (whole - 1) * T : p.L;
  return p;
}
// place in the sequence of the v-th step the block runs
__device__ __forceinline__ long long real_pos(const Piece& p, int v) {
  if (v < p.A) return p.begin + v;
  if (v < p.A + p.head) return p.begin + (p.L - p.head) + (v - p.A);
  return p.begin + p.A + (v - p.A - p.head);
}
// steps of the segment (a run within one tile) that starts at running step v
__device__ __forceinline__ int seg_len(const Piece& p, int v) {
  const int k0 = (int)(real_pos(p, v) % p.T);
  const int limit = v < p.A ? p.A - v : (v < p.A + p.head ? p.A + p.head - v : p.L - v);
  return (p.T - k0) < limit ? (p.T - k0) : limit;
}

__global__ void __launch_bounds__(SK_THREADS, 1) gemm_stream_k_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                   const __grid_constant__ CUtensorMap map_x, const SkArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the ring of stages starts on a 1024-byte boundary (the swizzle pattern repeats every 1024 bytes)
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int a_bytes = TILE_ROWS * KSTEP * 2;          // one box of W
  const int b_bytes = a.mpad * KSTEP * 2;             // one box of x (a multiple of 2048)
  const int KSUB = a.ksub;
  const int stage_bytes = KSUB * (a_bytes + b_bytes);
  float* part = reinterpret_cast<float*>(smem + (size_t)a.stages * stage_bytes);   // [mpad][128], the epilogue's
  __shared__ __align__(8) unsigned long long bars[2 * MAX_STAGES + 4];   // full[s], empty[s], acc_full[2], acc_empty[2]
  __shared__ uint32_t tmem_base_slot;
  __shared__ volatile int failed;
  __shared__ int s_epoch;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x, blocks = gridDim.x;
  const long long begin = piece_begin(a, b, blocks), end = piece_begin(a, b + 1, blocks);
  const int T = a.steps_per_tile;
  const int rows_out = a.swiglu ? 64 : TILE_ROWS;    // output columns a tile makes
  const uint32_t full0 = s2u(&bars[0]), empty0 = s2u(&bars[MAX_STAGES]);
  const uint32_t acc_full0 = s2u(&bars[2 * MAX_STAGES]), acc_empty0 = s2u(&bars[2 * MAX_STAGES + 2]);
  // running step v: boxes of W and of x into stage v % stages
  const Piece piece = make_piece(begin, end, T);
  const int L = piece.L;
  auto issue = [&](int v) {
    const long long pos = real_pos(piece, v);
    const int s = v % a.stages;
    const int tile = (int)(pos / T), kstep = (int)(pos % T);
    const int n0 = tile * rows_out;
    const uint32_t dst0 = s2u(smem + (size_t)s * stage_bytes);
    mbar_expect_tx(full0 + 8 * s, (uint32_t)stage_bytes);
    for (int sub = 0; sub < KSUB; ++sub) {
      const int kc = (kstep * KSUB + sub) * KSTEP;     // past K the boxes are filled with zeros
      const uint32_t dst = dst0 + sub * a_bytes;
      if (a.swiglu) {
        tma_load_2d(dst, &map_w, kc, n0, full0 + 8 * s);                           // 64 gate rows
        tma_load_2d(dst + 64 * KSTEP * 2, &map_w, kc, a.n_up + n0, full0 + 8 * s);  // their 64 up rows
      } else {
        tma_load_2d(dst, &map_w, kc, n0, full0 + 8 * s);
      }
      tma_load_2d(dst0 + KSUB * a_bytes + sub * b_bytes, &map_x, kc, 0, full0 + 8 * s);
    }
  };
  if (tid == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full0 + 8 * i, 1);
      mbar_init(acc_empty0 + 8 * i, 4);     // one arrival per epilogue warp
    }
    failed = 0;
    s_epoch = ld_acquire(a.flags) + 1;   // this launch's number (the launch before has ended: stream order)
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
  }
  if (warp == 1) tmem_alloc(s2u(&tmem_base_slot), a.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int epoch = s_epoch;

  if (warp == 0) {
    if (lane == 0) {
      // producer: the steps of the piece without a pause at tile borders
      int issued = 0;
      for (int v = 0; v < L; ++v, ++issued) {
        const int s = v % a.stages;
        if (v >= a.stages && !mbar_wait(empty0 + 8 * s, ((v / a.stages) - 1) & 1)) {
          failed = 1;
          break;
        }
        issue(v);
      }
      if (failed) {
        // copies that were asked for still write to this block's shared memory: wait for them (bounded)
        const int n = issued < a.stages ? issued : a.stages;
        for (int j = 0; j < n; ++j) {
          const int i = issued - 1 - j;
          mbar_wait(full0 + 8 * (i % a.stages), (i / a.stages) & 1);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // MMA issuer: segment j of the piece (the steps of one tile) adds up in accumulator j & 1
      const uint32_t idesc = instr_desc_bf16(TILE_ROWS, a.mpad);
      int seg = 0;
      for (int v = 0; v < L && !failed; ++seg) {
        const int len = seg_len(piece, v);
        const int buf = seg & 1, use = seg >> 1;
        if (use >= 1 && !mbar_wait(acc_empty0 + 8 * buf, (use - 1) & 1)) {
          failed = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * a.mpad);
        for (int j = 0; j < len; ++j) {
          const int i = v + j, s = i % a.stages;
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
              umma(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (j > 0 || sub > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);      // the stage is free once these MMAs have read it
        }
        if (failed) break;
        umma_commit(acc_full0 + 8 * buf);   // the segment's sum is complete once everything issued is done
        v += len;
      }
    }
  } else {
    // epilogue warps: warp w reads the 32 lanes of tensor memory it may read, (w % 4) * 32 ...
    const int et = tid - 64;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;               // row of D = row of the W tile
    int seg = 0;
    bool good = true;
    for (int v = 0; v < L; ++seg) {
      const long long pos = real_pos(piece, v);
      const int tile = (int)(pos / T), k0 = (int)(pos % T);
      const int len = seg_len(piece, v);
      const int buf = seg & 1, use = seg >> 1;
      const bool owner = k0 == 0;                      // the head of the tile: this block stores it
      if (good && !mbar_wait(acc_full0 + 8 * buf, use & 1)) good = false;
      if (failed) good = false;
      tc_fence_after();
      float* dst = owner ? part : a.ws + (size_t)b * a.mpad * TILE_ROWS;
      if (good) {
        for (int c0 = 0; c0 < a.mpad; c0 += 16) {
          float v[16];
          tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * a.mpad + c0), v);
#pragma unroll
          for (int i = 0; i < 16; ++i) dst[(size_t)(c0 + i) * TILE_ROWS + row] = v[i];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);   // the accumulator may be used again
      if (!owner) {
        __threadfence();
        epi_sync();
        if (et == 0 && good) st_release(a.flags + 2 + b, epoch);
        v += len;
        continue;
      }
      // the blocks after this one that hold the rest of the tile
      int n_others = 0;
      if (len < T) {
        const long long tile_end = (long long)(tile + 1) * T;
        while (b + 1 + n_others < blocks && piece_begin(a, b + 1 + n_others, blocks) < tile_end) ++n_others;
        for (int c = et; c < n_others; c += EPI_THREADS)
          if (!flag_wait(a.flags + 2 + b + 1 + c, epoch)) failed = 1;
      }
      epi_sync();
      if (failed) good = false;
      // the partials of the other blocks are added to this block's sum in block order, eight 16-byte
      // loads of a thread asked for together
      if (good && n_others > 0) {
        const int n4 = a.M * TILE_ROWS / 4;
        float4* part4 = reinterpret_cast<float4*>(part);
        for (int c = 0; c < n_others; ++c) {
          const float4* src4 = reinterpret_cast<const float4*>(a.ws + (size_t)(b + 1 + c) * a.mpad * TILE_ROWS);
          for (int i0 = et; i0 < n4; i0 += 8 * EPI_THREADS) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int i = i0 + j * EPI_THREADS;
              v[j] = i < n4 ? __ldcg(src4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int i = i0 + j * EPI_THREADS;
              if (i < n4) {
                float4 p = part4[i];
                p.x += v[j].x; p.y += v[j].y; p.z += v[j].z; p.w += v[j].w;
                part4[i] = p;
              }
            }
          }
        }
        epi_sync();
      }
      // eight output columns of one token at a time: this block's sum, then the partials in block order
      const int n0 = tile * rows_out;
      const int groups = rows_out / 8;
      for (int item = et; item < groups * a.M && good; item += EPI_THREADS) {
        const int m = item / groups, r = (item % groups) * 8;
        const float* src = part + (size_t)m * TILE_ROWS + r;
        float4 t0 = *reinterpret_cast<const float4*>(src), t1 = *reinterpret_cast<const float4*>(src + 4);
        float y[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
        float u[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (a.swiglu) {
          t0 = *reinterpret_cast<const float4*>(src + 64);
          t1 = *reinterpret_cast<const float4*>(src + 68);
          u[0] = t0.x; u[1] = t0.y; u[2] = t0.z; u[3] = t0.w; u[4] = t1.x; u[5] = t1.y; u[6] = t1.z; u[7] = t1.w;
        }
        const int n = n0 + r;
        if (n < (a.swiglu ? a.n_up : a.N)) {     // N and the first up row are multiples of 8: a group is in or out as a whole
          if (a.swiglu) {
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = y[i] / (1.f + expf(-y[i])) * u[i];
          }
          if (a.out_f32) {
            float* o = (float*)a.out + (size_t)m * a.ldc + n;
            *reinterpret_cast<float4*>(o) = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(y[4], y[5], y[6], y[7]);
          } else {
            uint4 st;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(y[0], y[1]), p1 = __floats2bfloat162_rn(y[2], y[3]),
                           p2 = __floats2bfloat162_rn(y[4], y[5]), p3 = __floats2bfloat162_rn(y[6], y[7]);
            st.x = *reinterpret_cast<uint32_t*>(&p0);
            st.y = *reinterpret_cast<uint32_t*>(&p1);
            st.z = *reinterpret_cast<uint32_t*>(&p2);
            st.w = *reinterpret_cast<uint32_t*>(&p3);
            *reinterpret_cast<uint4*>((__nv_bfloat16*)a.out + (size_t)m * a.ldc + n) = st;
          }
        }
      }
      epi_sync();     // the next segment writes over the shared-memory copy
      v += len;
    }
    if ((!good || failed) && et == 0) dk_report(a.err, DK_DEV_TIMEOUT, b, (int)begin, (int)(end - begin));
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, a.tmem_cols);
  // the last block to get here counts the launch number up for the next launch
  if (tid == 0) {
    __threadfence();
    int* done = a.flags + 1;
    if (atomicAdd(done, 1) == blocks - 1) {
      *done = 0;
      __threadfence();
      st_release(a.flags, epoch);
    }
  }
}
}  // namespace

namespace {
constexpr int FLAG_BYTES = 4096;   // head of the workspace: launch number, blocks done, one flag per block
int sm_count() { return dk_sm_count(); }
}  // namespace

extern "C" int dk_gemm_stream_k_supported(int M, int N, int K, int swiglu) {
  if (M < 1 || M > 128 || K < 64 || (K % 8) != 0) return 0;
  if (swiglu) {
    if ((N % 2) != 0 || ((N / 2) % 64) != 0) return 0;
  } else if ((N % 8) != 0) {
    return 0;
  }
  return 1;
}

// Bytes of workspace the kernel needs for M rows on this device (partials of every block, flags);
// it must be zero before its first use and is then kept between launches of one stream.
extern "C" long long dk_gemm_stream_k_workspace_bytes(int M) {
  const int mpad = (M + 15) / 16 * 16;
  return FLAG_BYTES + (long long)sm_count() * mpad * TILE_ROWS * 4;
}

// out_dtype DK_BF16 or DK_F32.  workspace: dk_gemm_stream_k_workspace_bytes(M) bytes, 256-byte aligned.
extern "C" int dk_gemm_stream_k(const void* x, const void* W, void* out, int M, int N, int K, int lda, int ldw, int ldc,
                                int out_dtype, int swiglu, void* workspace, int* err, cudaStream_t stream) {
  DK_REQUIRE(dk_gemm_stream_k_supported(M, N, K, swiglu), "gemm_stream_k: sizes not taken: M=%d N=%d K=%d swiglu=%d", M, N, K, swiglu);
  DK_REQUIRE((lda % 8) == 0 && (ldw % 8) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)W % 16) == 0,
             "gemm_stream_k: operands must start on 16-byte boundaries with leading sizes that are multiples of 8");
  DK_REQUIRE(out_dtype == DK_BF16 || out_dtype == DK_F32, "gemm_stream_k: unknown output dtype %d", out_dtype);
  DK_REQUIRE((ldc % 8) == 0 && ((uintptr_t)out % 16) == 0,
             "gemm_stream_k: the output must start on a 16-byte boundary with a leading size that is a multiple of 8");
  DK_REQUIRE(workspace != nullptr && ((uintptr_t)workspace % 256) == 0, "gemm_stream_k: the workspace must be 256-byte aligned");
  SkArgs a;
  a.out = out;
  a.err = err;
  a.M = M; a.N = N; a.K = K; a.ldc = ldc;
  a.mpad = (M + 15) / 16 * 16;
  a.out_f32 = out_dtype == DK_F32;
  a.swiglu = swiglu;
  a.n_up = swiglu ? N / 2 : 0;
  a.tmem_cols = 32;
  while (a.tmem_cols < 2 * a.mpad) a.tmem_cols *= 2;       // two accumulators of mpad columns
  const int sms = sm_count();
  DK_REQUIRE((sms + 2) * 4 <= FLAG_BYTES, "gemm_stream_k: %d SMs are more than the flags have room for", sms);
  a.flags = reinterpret_cast<int*>(workspace);     // at a fixed place, whatever the number of rows
  a.ws = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + FLAG_BYTES);
  const int a_bytes = TILE_ROWS * KSTEP * 2;
  const int b_bytes = a.mpad * KSTEP * 2;
  const int part_bytes = a.mpad * TILE_ROWS * 4;
  a.ksub = 2;
  const int stage_bytes = a.ksub * (a_bytes + b_bytes);
  int stages = (226 * 1024 - 1024 - part_bytes) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  DK_REQUIRE(stages >= 2, "gemm_stream_k: M=%d leaves no room for two stages", M);
  a.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + part_bytes + 1024;
  const int rows_out = swiglu ? 64 : TILE_ROWS;
  const int n_out = swiglu ? N / 2 : N;
  a.tiles = (n_out + rows_out - 1) / rows_out;
  a.steps_per_tile = (K + KSTEP * a.ksub - 1) / (KSTEP * a.ksub);
  a.total = (long long)a.tiles * a.steps_per_tile;
  const int blocks = (long long)sms < a.total ? sms : (int)a.total;
  CUtensorMap map_w, map_x;
  DK_REQUIRE(make_tensor_map_bf16(&map_w, W, N, K, ldw, swiglu ? 64 : TILE_ROWS), "gemm_stream_k: cannot encode the tensor map of W");
  DK_REQUIRE(make_tensor_map_bf16(&map_x, x, M, K, lda, a.mpad), "gemm_stream_k: cannot encode the tensor map of x");
  static size_t configured_on[DK_MAX_DEVICES] = {0};
  size_t& configured = configured_on[dk_current_device()];
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      dk_set_error("gemm_stream_k: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return DK_ERR_LAUNCH;
    }
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks, 1, 1);
  cfg.blockDim = dim3(SK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // the blocks wait for one another: all resident, or no launch
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_k_kernel, map_w, map_x, a);
  if (e != cudaSuccess) {
    dk_set_error("gemm_stream_k: launch failed: %s", cudaGetErrorString(e));
    return DK_ERR_LAUNCH;
  }
  return dk_check_launch("gemm_stream_k");
}
