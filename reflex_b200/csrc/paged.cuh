// Addressing of the paged key/value store.
//
// A cache entry (one per caching layer run) is an array of pages
// [n_pages][n_kv_heads][PAGE][head_dim]; a sequence's positions map to pages
// through its slot's row of the page table: position p lives in page
// table[slot * max_pages + p / PAGE] at token p % PAGE.  One (page, kv head)
// tile is PAGE * head_dim contiguous elements.
#pragma once
#include <stddef.h>

namespace rfx {

struct PagedKV {
    const int* page_table;  // [slots][max_pages]
    int max_pages;
    int page_size;   // tokens per page
    int n_kv_heads;
    int head_dim;
};

__device__ __forceinline__ size_t kv_offset(const PagedKV& c, int slot, int pos, int kvh) {
    const int page = c.page_table[(size_t)slot * c.max_pages + pos / c.page_size];
    return (((size_t)page * c.n_kv_heads + kvh) * c.page_size + (pos % c.page_size)) *
           (size_t)c.head_dim;
}

}  // namespace rfx
