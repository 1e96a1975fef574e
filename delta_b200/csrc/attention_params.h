// Arguments of the paged attention kernels.  The Python side mirrors this
// struct field by field; dk_sizeof_attn_params() lets it check the size.
#pragma once
#include <stdint.h>

struct DkAttnParams {
  const void* q;           // [T, q_stride] elements; head h of token t at q + t*q_stride + h*hd
  void* out;               // [T, H*hd]
  const void* kv;          // cache of this layer: [num_pages, 2, KV, ps, hd]
  const int* block_table;  // [rows, max_pages] physical page of logical page j, per batch row
  const int* tok_row;      // [T] batch row of each token
  const int* tok_pos;      // [T] position of each token in its request
  const int* row_slot;     // [rows] request slot of each batch row
  const int* row_flags;    // [rows] bit 0: a decode row that page selection applies to
  const int* row_q_start;  // [rows] first token of the row in this step
  const int* row_q_len;    // [rows] tokens of the row in this step
  const int* row_pos_start;// [rows] position of the row's first token
  const int* sel_pages;    // [slots, sel_stride] chosen logical pages, ascending; or null
  const int* sel_count;    // [slots] how many are chosen, -1: read everything; or null
  float* dump;             // [rows, H, dump_stride] scaled scores of flagged rows; or null
  float* lse;              // [T, H] log-sum-exp of each (token, head); or null
  void* scratch;           // partial results of kernels that split the keys; or null
  int* err;                // device error record, 4 ints; or null
  const float* rope_table; // decode kernel with fuse != 0: cos/sin [positions, hd/2, 2]; null: no rotation
  int T, rows, H, KV, hd, ps, max_pages, num_pages;
  int q_stride, window, sel_stride, dump_stride, dtype, splits;
  float scale;
  int block_entries;       // set by the launchers: pages one block keeps in shared memory
  int row_filter;          // 0: every row; 1: only rows that bring one token; 2: only rows that bring more
  int fuse;                // decode kernel: q points into rows [q | k | v] that are not rotated yet; the kernel rotates
                           // q and k itself and (fuse == 2) appends k and v of the new token to its page
  int rope_positions;      // rows of rope_table
  int reserved;            // bit 0 (decode kernel): the pages of the rows lie scattered over the pool, do not look for runs;
                           // bit 1 (decode kernel, 2..8 splits): the splits of a (row, kv head) are launched as one cluster and
                           // merge through distributed shared memory (no scratch buffer, no merge kernel)
};
