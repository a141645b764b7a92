// What the latent-attention kernels share: where a token's row lies in a page.
//
// Cache layout (one page of one cache entry): [position in page][kr + rot]: the token's normed latent (kr numbers,
// from which every head's keys and values are linear maps) followed by the rotated key part that all heads share.
// There is one such row per token whatever the number of heads.
#pragma once
#include "common.cuh"

struct LatentCache {
    int max_pages, page_size, kr, rot;
    long long page_stride;      // elements between consecutive pages of this entry
    long long entry_offset;     // elements from the pool's start to this entry's part of page 0
};

template <typename T>
__device__ __forceinline__ T* latent_row(T* pool, const LatentCache& c, int page, int pip) {
    return pool + c.entry_offset + (long long)page * c.page_stride + (long long)pip * (c.kr + c.rot);
}
