// Arguments shared by the attention kernels (see attention_generic.cu for the meaning of a
// tile: ROWS query rows of one request and one kv head, a row being a (token, head) pair).
#pragma once

namespace fsie {

struct AttnParams {
    const void* q; int q_ld;                 // [tokens, q_ld]; head h of token t at t*q_ld + h*head_dim
    const void* k_pages; const void* v_pages;
    long long page_stride; int page_size;    // elements between pages; slots per page
    const int* block_tables; int bt_stride;  // [items, bt_stride] page ids (-1 = released)
    const int* tile_item; const int* tile_row0;   // [tiles]
    const int* item_qstart; const int* item_qlen; const int* item_pos0;   // [items]
    void* out; int out_ld;                   // [tokens, out_ld]
    float* part_o; float* part_ml;           // [nsplit, tokens, heads, head_dim], [nsplit, tokens, heads, 2]
    int tokens, heads, kv_heads, head_dim, window, nsplit;
    float scale;
};

}  // namespace fsie
