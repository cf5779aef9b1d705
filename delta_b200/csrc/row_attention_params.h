// Arguments of the paged attention kernels over a cache of rows: every cached token of a key-value head is
// one row of `row_width` elements that holds its key at `k_off` (dk elements) and its value at `v_off`
// (dv elements).  Key and value may have different sizes, lie side by side, or overlap: a latent cache
// whose value is the front part of its key is k_off = v_off = 0 with dv < dk and one key-value head.
// A page of a layer is [KV][ps][row_width].  The Python side mirrors this struct field by field.
#pragma once
#include <stdint.h>

struct DkRowAttnParams {
  const void* q;            // head h of token t at q + t*q_stride + h*q_head_stride, dk elements
  void* out;                // [T, H*dv]
  const void* cache;        // [num_pages, KV, ps, row_width]
  const int* block_table;   // [rows, max_pages]
  const int* tok_row;       // [T]
  const int* tok_pos;       // [T]
  const int* row_q_start;   // [rows] first token of the row in this step
  const int* row_q_len;     // [rows] tokens of the row in this step
  const int* row_pos_start; // [rows] position of the row's first token
  const float* sink;        // [H] a logit that joins every softmax denominator with no value; or null
  const float* dist_bias;   // [H, dist_max + 1] added to the score of query i and key j: entry min(i - j, dist_max) of the head's row; or null
  void* scratch;            // partial results of kernels that split the keys; or null
  int* err;                 // device error record, 4 ints; or null
  int T, rows, H, KV, dk, dv, ps, max_pages, num_pages;
  int q_stride, q_head_stride, row_width, k_off, v_off;
  int window;               // > 0: position i sees keys j with i - window < j <= i
  int dtype;
  int splits;               // decode kernel: blocks that share the keys of a (row, key-value head)
  int row_filter;           // 0: every row; 1: only rows that bring one token; 2: only rows that bring more
  float scale;
  float softcap;            // > 0: the scaled score s becomes softcap * tanh(s / softcap) (before the distance bias)
  int dist_max;             // last entry of a row of dist_bias: every distance from here on takes it
  int reserved;
};
