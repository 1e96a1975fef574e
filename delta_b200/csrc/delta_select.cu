// DELTA's selective cache: the recency window a step starts with, the page score
// from the dumped scores of a planner layer, and the top-k page selection.
//
// State per request slot: sel_pages[slot][0..k) = chosen logical pages in
// ascending order, sel_count[slot] = how many (-1: the request reads everything).
#include "common.cuh"

namespace {

// A request with n pages uses the subset when n / min(n, k) > ratio
// (reference, per batch: backend.py:1893-1897).
//
// How many pages a request of `seq` tokens counts: those it holds, ceil(seq / ps); with
// `ahead` one more once the newest page is exactly full, as the reference does, which
// takes a request's next page before the token that needs it (scheduler.py:60-74).
// That page holds no key: it scores zero, it can be chosen (it is the newest page, so it
// is among the last L), and it is left out of what the attention reads.
__device__ __forceinline__ int pages_counted(int seq, int ps, int ahead) { return ahead ? seq / ps + 1 : (seq + ps - 1) / ps; }

__device__ __forceinline__ bool selection_active(int n_pages, int k, double ratio) {
  const int sub = n_pages < k ? n_pages : k;
  return sub > 0 && (double)n_pages / (double)sub > ratio;
}

// Before a planner has run in a step the subset is the last k pages
// (reference: backend.py:1871-1873, 2054-2055).
__global__ void recent_pages_kernel(const int* __restrict__ row_slot, const int* __restrict__ row_flags,
                                    const int* __restrict__ row_pos_start, const int* __restrict__ row_q_len,
                                    int* __restrict__ sel_pages, int* __restrict__ sel_count, int k, int ps, double ratio,
                                    int ahead) {
  const int b = blockIdx.x;
  const int slot = row_slot[b];
  const int seq = row_pos_start[b] + row_q_len[b];
  const int n = pages_counted(seq, ps, ahead), held = (seq + ps - 1) / ps;
  const bool active = (row_flags[b] & 1) && selection_active(n, k, ratio);
  const int count = k - (n - held);
  if (threadIdx.x == 0) sel_count[slot] = active ? count : -1;
  if (active)
    for (int i = threadIdx.x; i < count; i += blockDim.x) sel_pages[(size_t)slot * k + i] = n - k + i;
}

// score[row][j] = sum over the tokens t of page j of max_h exp(z[row,h,t] - lse[h])
// = sum of the head-wise maximum of the softmax (reference: backend.py:887-904;
// the softmax is rebuilt from the log-sum-exp as at backend.py:855-885).
__global__ void __launch_bounds__(128) page_scores_kernel(const float* __restrict__ dump, const float* __restrict__ lse,
                                                          const int* __restrict__ row_flags, const int* __restrict__ row_q_start,
                                                          const int* __restrict__ row_pos_start, const int* __restrict__ row_q_len,
                                                          float* __restrict__ scores, int H, int ps, int dump_stride,
                                                          int max_pages, int k, double ratio, int ahead) {
  __shared__ float part[128];
  const int b = blockIdx.y, j = blockIdx.x;
  const int seq = row_pos_start[b] + row_q_len[b];
  const int held = (seq + ps - 1) / ps;
  if (!(row_flags[b] & 1) || !selection_active(pages_counted(seq, ps, ahead), k, ratio) || j >= held) return;
  const int t = row_q_start[b] + row_q_len[b] - 1;
  const int tok = threadIdx.x % ps, hg = threadIdx.x / ps, n_hg = 128 / ps;
  const int key = j * ps + tok;
  float mx = 0.f;
  if (key < seq && key < dump_stride) {
    for (int h = hg; h < H; h += n_hg) {
      const float z = dump[((size_t)b * H + h) * dump_stride + key];
      mx = fmaxf(mx, expf(z - lse[(size_t)t * H + h]));
    }
  }
  part[threadIdx.x] = mx;
  __syncthreads();
  if (threadIdx.x < ps) {
    float v = part[threadIdx.x];
    for (int g = 1; g < n_hg; ++g) v = fmaxf(v, part[g * ps + threadIdx.x]);
    part[threadIdx.x] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < ps; ++i) s += part[i];
    scores[(size_t)b * max_pages + j] = s;
  }
}

// One top-k per request (reference: page_selector_v2.py:113-150): NaN and -inf
// become -inf, a bias of -bias*j is added, the last `keep_last` pages get +inf,
// the k best are kept and written in ascending page order.  Equal scores go to
// the older page.
__global__ void select_pages_kernel(const float* __restrict__ scores, const int* __restrict__ row_slot,
                                    const int* __restrict__ row_flags, const int* __restrict__ row_pos_start,
                                    const int* __restrict__ row_q_len, int* __restrict__ sel_pages, int* __restrict__ sel_count,
                                    int max_pages, int k, int keep_last, int ps, float bias, double ratio, int ahead) {
  extern __shared__ float sm[];
  float* sc = sm;
  int* chosen = (int*)(sm + max_pages + 1);
  const int b = blockIdx.x;
  const int seq = row_pos_start[b] + row_q_len[b];
  const int n = pages_counted(seq, ps, ahead), held = (seq + ps - 1) / ps;
  if (!(row_flags[b] & 1) || !selection_active(n, k, ratio)) return;
  const int slot = row_slot[b];
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float s = j < held ? scores[(size_t)b * max_pages + j] : 0.f;
    if (isnan(s) || s == -INFINITY) s = -INFINITY;
    s = __fadd_rn(s, __fmul_rn(-(float)j, bias));
    if (j >= n - keep_last) s = INFINITY;
    sc[j] = s;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const float mine = sc[j];
    int rank = 0;
    for (int i = 0; i < n; ++i) {
      const float o = sc[i];
      rank += (o > mine || (o == mine && i < j)) ? 1 : 0;
    }
    chosen[j] = rank < k ? 1 : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = 0, taken = 0;
    for (int j = 0; j < n && taken < k; ++j)
      if (chosen[j]) {
        ++taken;
        if (j < held) sel_pages[(size_t)slot * k + c++] = j;
      }
    sel_count[slot] = c;
  }
}
}  // namespace

extern "C" int dk_recent_pages(const int* row_slot, const int* row_flags, const int* row_pos_start, const int* row_q_len,
                               int* sel_pages, int* sel_count, int rows, int k, int ps, double ratio, int ahead,
                               cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && k > 0 && ps > 0, "recent_pages: bad sizes rows=%d k=%d ps=%d", rows, k, ps);
  recent_pages_kernel<<<rows, 128, 0, stream>>>(row_slot, row_flags, row_pos_start, row_q_len, sel_pages, sel_count, k, ps, ratio, ahead);
  return dk_check_launch("recent_pages");
}

extern "C" int dk_page_scores(const float* dump, const float* lse, const int* row_flags, const int* row_q_start,
                              const int* row_pos_start, const int* row_q_len, float* scores, int rows, int H, int ps,
                              int dump_stride, int max_pages, int k, double ratio, int ahead, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && H > 0 && max_pages > 0, "page_scores: bad sizes");
  DK_REQUIRE(ps >= 1 && ps <= 128 && (ps & (ps - 1)) == 0, "page_scores: page size %d must be a power of two <= 128", ps);
  DK_REQUIRE(rows <= 65535, "page_scores: too many rows");
  dim3 grid(max_pages, rows);
  page_scores_kernel<<<grid, 128, 0, stream>>>(dump, lse, row_flags, row_q_start, row_pos_start, row_q_len, scores, H, ps,
                                               dump_stride, max_pages, k, ratio, ahead);
  return dk_check_launch("page_scores");
}

extern "C" int dk_select_pages(const float* scores, const int* row_slot, const int* row_flags, const int* row_pos_start,
                               const int* row_q_len, int* sel_pages, int* sel_count, int rows, int max_pages, int k,
                               int keep_last, int ps, float bias, double ratio, int ahead, cudaStream_t stream) {
  if (rows == 0) return 0;
  DK_REQUIRE(rows > 0 && max_pages > 0 && k > 0, "select_pages: bad sizes");
  DK_REQUIRE(keep_last >= 1 && keep_last <= k, "select_pages: keep_last %d must lie in 1..k=%d", keep_last, k);
  DK_REQUIRE(max_pages <= 4096, "select_pages: %d pages per request are above the 4096 this kernel ranks in shared memory", max_pages);
  const size_t smem = (size_t)(max_pages + 1) * (sizeof(float) + sizeof(int));
  select_pages_kernel<<<rows, 256, smem, stream>>>(scores, row_slot, row_flags, row_pos_start, row_q_len, sel_pages, sel_count,
                                                   max_pages, k, keep_last, ps, bias, ratio, ahead);
  return dk_check_launch("select_pages");
}
