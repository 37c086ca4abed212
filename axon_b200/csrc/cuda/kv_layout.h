// The record a caller passes for a paged cache: where one layer's keys and values lie in
// its page pool, and which block table maps a request's positions to pages.  Every
// launcher that reads or writes the cache takes a pointer to one.
//
// Pool layout: pool[page][entry][plane 0: keys | plane 1: values], a plane being
// [kv_head][page_size][row width].  Keys are `head_dim` wide and values `v_dim` wide
// (equal for ordinary attention).  With `planes` == 1 there is one plane per entry: a
// mixer that keeps a single latent row per position; kernels then read values from the
// key plane (v_offset 0, v_dim == head_dim).
#pragma once

#include <stdint.h>

struct AxonKvLayout {
    const int32_t* block_table;  // [slots][table_stride]: logical page -> physical page
    int32_t table_stride;
    int32_t page_size;
    int32_t kv_heads;
    int32_t head_dim;            // elements of a key row
    int64_t page_stride;         // elements between two pages of the pool
    int64_t entry_offset;        // elements from a page's start to this layer's key plane
    int64_t v_offset;            // elements from the key plane to the value plane
    int32_t v_dim;               // elements of a value row
    int32_t planes;              // 2 (keys and values) or 1
    // Checked tables (a debugging mode): with `fault` set, every block-table entry a kernel
    // reads is compared with `n_pages` (the sink page's index, the largest valid entry); a
    // larger or negative one is not followed: the kernel reads or writes the sink page
    // instead, sets fault[0] = 1 and fault[1] = the entry.  Null switches the check off.
    int32_t n_pages;
    int32_t reserved;
    uint32_t* fault;
};
