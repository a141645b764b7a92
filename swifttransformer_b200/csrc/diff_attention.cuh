// What the differential-attention kernels share: where an entry's keys and values lie in a page, and which
// keys a query sees.
//
// Cache layout (one page of one cache entry; kd = 2 * dim, the two maps' keys side by side):
//   keys   [kv_head][position in page][kd]     at offset 0
//   values [kv_head][position in page][vd]     at offset nkv * page_size * kd
#pragma once
#include "common.cuh"

struct DiffCache {
    int max_pages, page_size, nkv, kd, vd;
    long long page_stride;      // elements between consecutive pages of this entry
    long long entry_offset;     // elements from the pool's start to this entry's part of page 0
};

template <typename T>
__device__ __forceinline__ T* cache_keys(T* pool, const DiffCache& c, int page, int kvh, int pip) {
    return pool + c.entry_offset + (long long)page * c.page_stride + ((long long)kvh * c.page_size + pip) * c.kd;
}
template <typename T>
__device__ __forceinline__ T* cache_values(T* pool, const DiffCache& c, int page, int kvh, int pip) {
    return pool + c.entry_offset + (long long)page * c.page_stride + (long long)c.nkv * c.page_size * c.kd +
           ((long long)kvh * c.page_size + pip) * c.vd;
}

__device__ __forceinline__ int first_visible(int pos, int block, int window) {
    if (block > 0) return (pos / block) * block;
    if (window > 0) return max(0, pos - window + 1);
    return 0;
}

__device__ __forceinline__ float soft_cap(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

