// Paged prefill attention for bfloat16: rows that bring more than one token (portions of
// prompts), causal, over the block table.
//
// Grid (query tiles of 64 tokens, heads, batch rows); 4 warps per block, 16 query rows per
// warp.  Keys and values of the row's pages stream through shared memory in tiles of 64
// keys (cp.async, two stages, 16-byte chunks swizzled for ldmatrix).  Per tile and warp:
// S = Q K^T (mma.sync.m16n8k16, float accumulators), mask by position (causal, window),
// online softmax in float, O += P V.  The queries' own keys were appended before this
// kernel runs, so a portion of a prompt attends to the cache and to itself alike, and the
// result does not depend on where a prompt was cut.
//
// Rows that bring one token are left to the decode kernel (row_filter 2); with row_filter 0
// this kernel takes them too.
#include "common.cuh"
#include "attention_params.h"
#include "mma_helpers.cuh"

namespace {
constexpr int QT = 64;       // queries per block
constexpr int KT = 64;       // keys per tile
constexpr int PSTAGES = 2;
constexpr int PWARPS = 4;
constexpr int PTHREADS = PWARPS * 32;

template <int HD>
__global__ void __launch_bounds__(PTHREADS) attention_prefill_kernel(const DkAttnParams p) {
  constexpr int CHUNKS = HD / 8;
  constexpr int ROW_BYTES = HD * 2;
  constexpr int TILE_BYTES = KT * ROW_BYTES;
  constexpr int KB = HD / 16;
  constexpr int NT = HD / 8;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* kv_smem = smem;                                          // PSTAGES * 2 * TILE_BYTES
  int* s_page = reinterpret_cast<int*>(smem + PSTAGES * 2 * TILE_BYTES);   // physical page of each entry

  const int row = blockIdx.z, h = blockIdx.y;
  const int q_len = p.row_q_len[row];
  if (p.row_filter == 2 && q_len == 1) return;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;   // late tiles have the most keys: start them first
  const int q0 = qt * QT;
  if (q0 >= q_len) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int ps = p.ps, G = p.H / p.KV, kvh = h / G;
  const int nq = min(QT, q_len - q0);
  const int t0 = p.row_q_start[row] + q0;
  const int pos0 = p.row_pos_start[row] + q0;
  const int last_pos = pos0 + nq - 1;
  const int lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int first_page = lo / ps;
  const int n_entries = last_pos / ps - first_page + 1;
  if (n_entries > p.block_entries) {
    if (tid == 0) dk_report(p.err, DK_DEV_BAD_POSITION, t0, last_pos, p.max_pages * ps);
    return;
  }
  const __nv_bfloat16* kv = reinterpret_cast<const __nv_bfloat16*>(p.kv);
  for (int i = tid; i < n_entries; i += PTHREADS) {
    const int lp = first_page + i;
    int page = -1;
    if (lp < p.max_pages) {
      page = p.block_table[(size_t)row * p.max_pages + lp];
      if (page < 0 || page >= p.num_pages) {
        dk_report(p.err, DK_DEV_BAD_PAGE, t0, lp, page);
        page = -1;
      }
    }
    s_page[i] = page;
  }
  __syncthreads();
  const int pages_per_tile = KT / ps;
  const int n_tiles = (n_entries + pages_per_tile - 1) / pages_per_tile;
  const int key_base = first_page * ps;     // position of key 0 of tile 0

  // this warp's 16 query rows as A fragments
  const int r0 = warp * 16 + g, r1 = r0 + 8;
  uint32_t qa[KB][4];
  {
    const __nv_bfloat16* q = reinterpret_cast<const __nv_bfloat16*>(p.q) + (size_t)h * HD;
    const __nv_bfloat16* qr0 = q + (size_t)(t0 + min(r0, nq - 1)) * p.q_stride;
    const __nv_bfloat16* qr1 = q + (size_t)(t0 + min(r1, nq - 1)) * p.q_stride;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      const int c = kb * 16 + 2 * tq;
      qa[kb][0] = *reinterpret_cast<const uint32_t*>(qr0 + c);
      qa[kb][1] = *reinterpret_cast<const uint32_t*>(qr1 + c);
      qa[kb][2] = *reinterpret_cast<const uint32_t*>(qr0 + c + 8);
      qa[kb][3] = *reinterpret_cast<const uint32_t*>(qr1 + c + 8);
    }
  }
  const int pos_r0 = pos0 + r0, pos_r1 = pos0 + r1;
  const int warp_first_pos = pos0 + warp * 16, warp_last_pos = min(pos0 + warp * 16 + 15, last_pos);

  auto load_tile = [&](int tile, int stage) {
    unsigned char* kdst = kv_smem + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* vdst = kdst + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < KT * CHUNKS / PTHREADS; ++i) {
      const int c = tid + i * PTHREADS;
      const int tok = c / CHUNKS, part = c % CHUNKS;
      const int el = tile * pages_per_tile + tok / ps, off = tok % ps;
      bool valid = false;
      size_t koff = 0;
      if (el < n_entries) {
        const int page = s_page[el];
        if (page >= 0 && key_base + tile * KT + tok <= last_pos) {
          valid = true;
          koff = ((((size_t)page * 2 + 0) * p.KV + kvh) * ps + off) * HD + part * 8;
        }
      }
      const int sw = (part ^ (tok & 7)) * 16;
      cp_async_16(smem_u32(kdst + tok * ROW_BYTES + sw), kv + koff, valid);
      cp_async_16(smem_u32(vdst + tok * ROW_BYTES + sw), kv + koff + (size_t)p.KV * ps * HD, valid);
    }
  };

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const float sc_log2 = p.scale * 1.4426950408889634f;

  load_tile(0, 0);
  cp_async_commit();
  for (int tile = 0; tile < n_tiles; ++tile) {
    if (tile + 1 < n_tiles) load_tile(tile + 1, (tile + 1) % PSTAGES);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int stage = tile % PSTAGES;
    const uint32_t kbase = smem_u32(kv_smem + (size_t)stage * 2 * TILE_BYTES);
    const uint32_t vbase = kbase + TILE_BYTES;
    const int kt0 = key_base + tile * KT;   // position of the tile's first key
    // a warp skips tiles that none of its rows can see
    const bool visible = warp * 16 < nq && kt0 <= warp_last_pos && (p.window <= 0 || kt0 + KT - 1 > warp_first_pos - p.window);
    if (visible) {
      float s[KT / 8][4];
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) {
        const int tok = j * 8 + (lane & 7);
#pragma unroll
        for (int kb = 0; kb < KB; kb += 2) {
          const int chunk = 2 * kb + (lane >> 3);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, kbase + tok * ROW_BYTES + ((chunk ^ (tok & 7)) * 16));
          mma_bf16(s[j], qa[kb], b0, b1);
          mma_bf16(s[j], qa[kb + 1], b2, b3);
        }
      }
      // mask by position, then the online softmax (log2 units)
      const bool need_mask = kt0 + KT - 1 > warp_first_pos || (p.window > 0 && kt0 <= warp_last_pos - p.window + 1) || kt0 < lo;
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int key = kt0 + j * 8 + 2 * tq + c;
          float v0 = s[j][c] * sc_log2, v1 = s[j][2 + c] * sc_log2;
          if (need_mask) {
            if (key > pos_r0 || (p.window > 0 && key <= pos_r0 - p.window)) v0 = -INFINITY;
            if (key > pos_r1 || (p.window > 0 && key <= pos_r1 - p.window)) v1 = -INFINITY;
          }
          s[j][c] = v0;
          s[j][2 + c] = v1;
          tmax[0] = fmaxf(tmax[0], v0);
          tmax[1] = fmaxf(tmax[1], v1);
        }
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
        const float m_new = fmaxf(m_run[r], tmax[r]);
        m_use[r] = m_new == -INFINITY ? 0.f : m_new;
        corr[r] = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
      }
#pragma unroll
      for (int kb2 = 0; kb2 < KT / 16; ++kb2) {
        uint32_t pa[4];
        {
          const float p00 = exp2f(s[2 * kb2][0] - m_use[0]), p01 = exp2f(s[2 * kb2][1] - m_use[0]);
          const float p02 = exp2f(s[2 * kb2][2] - m_use[1]), p03 = exp2f(s[2 * kb2][3] - m_use[1]);
          const float p10 = exp2f(s[2 * kb2 + 1][0] - m_use[0]), p11 = exp2f(s[2 * kb2 + 1][1] - m_use[0]);
          const float p12 = exp2f(s[2 * kb2 + 1][2] - m_use[1]), p13 = exp2f(s[2 * kb2 + 1][3] - m_use[1]);
          l_run[0] += p00 + p01 + p10 + p11;
          l_run[1] += p02 + p03 + p12 + p13;
          pa[0] = pack_bf16(p00, p01);
          pa[1] = pack_bf16(p02, p03);
          pa[2] = pack_bf16(p10, p11);
          pa[3] = pack_bf16(p12, p13);
        }
        const int tok = kb2 * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
          const int chunk = n + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(b0, b1, b2, b3, vbase + tok * ROW_BYTES + ((chunk ^ (tok & 7)) * 16));
          mma_bf16(o[n], pa, b0, b1);
          mma_bf16(o[n + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();   // every warp is done with this stage before the next load overwrites it
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)h * HD;
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  if (r0 < nq) {
    __nv_bfloat16* orow = out + (size_t)(t0 + r0) * p.H * HD;
#pragma unroll
    for (int n = 0; n < NT; ++n)
      *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * tq) = pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
    if (p.lse != nullptr && tq == 0)
      p.lse[(size_t)(t0 + r0) * p.H + h] = l_run[0] > 0.f ? m_run[0] * 0.6931471805599453f + logf(l_run[0]) : -INFINITY;
  }
  if (r1 < nq) {
    __nv_bfloat16* orow = out + (size_t)(t0 + r1) * p.H * HD;
#pragma unroll
    for (int n = 0; n < NT; ++n)
      *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * tq) = pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
    if (p.lse != nullptr && tq == 0)
      p.lse[(size_t)(t0 + r1) * p.H + h] = l_run[1] > 0.f ? m_run[1] * 0.6931471805599453f + logf(l_run[1]) : -INFINITY;
  }
}

template <int HD>
int launch(const DkAttnParams& pin, int max_q_len, cudaStream_t stream) {
  DkAttnParams p = pin;
  p.block_entries = p.max_pages;
  const size_t smem = (size_t)PSTAGES * 2 * KT * HD * 2 + (size_t)p.block_entries * sizeof(int);
  if (smem > 200 * 1024) {
    dk_set_error("attention_prefill: %d pages per request need more shared memory than a block has", p.max_pages);
    return DK_ERR_ARG;
  }
  static size_t configured_on[DK_MAX_DEVICES] = {0};
  size_t& configured = configured_on[dk_current_device()];
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      dk_set_error("attention_prefill: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
      return DK_ERR_LAUNCH;
    }
    configured = smem;
  }
  dim3 grid((max_q_len + QT - 1) / QT, p.H, p.rows);
  attention_prefill_kernel<HD><<<grid, PTHREADS, smem, stream>>>(p);
  return dk_check_launch("attention_prefill");
}
}  // namespace

extern "C" int dk_attention_prefill_supported(int dtype, int H, int KV, int hd, int ps) {
  if (dtype != DK_BF16 || KV <= 0 || H % KV != 0) return 0;
  if (hd != 64 && hd != 128) return 0;
  if (ps < 1 || ps > KT || (ps & (ps - 1)) != 0) return 0;
  return 1;
}

// max_q_len: the most tokens any row brings (sizes the grid).
extern "C" int dk_attention_prefill(const DkAttnParams* pp, int max_q_len, cudaStream_t stream) {
  const DkAttnParams& p = *pp;
  if (p.T == 0 || p.rows == 0) return 0;
  DK_REQUIRE(dk_attention_prefill_supported(p.dtype, p.H, p.KV, p.hd, p.ps),
             "attention_prefill: sizes not taken (bfloat16, head size 64 or 128, page size a power of two <= 64): "
             "dtype=%d H=%d KV=%d hd=%d ps=%d", p.dtype, p.H, p.KV, p.hd, p.ps);
  DK_REQUIRE(max_q_len >= 1, "attention_prefill: max_q_len must be positive");
  DK_REQUIRE(p.row_q_start && p.row_q_len && p.row_pos_start, "attention_prefill: row_q_start / row_q_len / row_pos_start are missing");
  DK_REQUIRE(p.H <= 65535 && p.rows <= 65535, "attention_prefill: grid too large");
  DK_REQUIRE(p.q_stride % 2 == 0, "attention_prefill: q stride must be even");
  return p.hd == 64 ? launch<64>(p, max_q_len, stream) : launch<128>(p, max_q_len, stream);
}
