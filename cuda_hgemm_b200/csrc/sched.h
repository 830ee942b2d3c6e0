// Work decomposition shared by host code and the kernels: tile rasterisation for L2 reuse,
// and the contiguous unit ranges ("stream-K") that let every SM get an equal share of
// k-blocks when the tile count does not fill the GPU.
//
// The reference maps blocks to tiles in 16-wide serpentine super-columns
// (src/mma/mma_async_stage4.cu:60-62); the grouped order below is the same idea with the
// group running along M and a width chosen per shape.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200 {

struct TileCoord {
    uint32_t m_blk;
    uint32_t n_blk;
};

// Linear tile id -> (m_blk, n_blk). Tiles are walked in bands of about `group_m` row blocks;
// inside a band the row block moves fastest, and odd bands walk the columns backwards so the
// column tiles at a band boundary are still in L2. The row blocks are spread evenly over the
// bands (59 row blocks at group_m = 8 give bands of 8,8,8,7,7,7,7,7, not seven of 8 and one of
// 3): a thin last band would make its waves long and narrow and lose the reuse of A.
B200_HD TileCoord tile_coord(uint32_t t, uint32_t m_blocks, uint32_t n_blocks, uint32_t group_m) {
    const uint32_t bands = (m_blocks + group_m - 1) / group_m;
    const uint32_t base = m_blocks / bands;   // rows of the shorter bands
    const uint32_t extra = m_blocks % bands;  // the first `extra` bands have one row more
    const uint32_t tall_tiles = extra * (base + 1) * n_blocks;
    uint32_t band, first_m, rows_here, r;
    if (t < tall_tiles) {
        rows_here = base + 1;
        band = t / (rows_here * n_blocks);
        first_m = band * rows_here;
        r = t - band * rows_here * n_blocks;
    } else {
        rows_here = base;
        const uint32_t u = t - tall_tiles;
        const uint32_t b = u / (rows_here * n_blocks);
        band = extra + b;
        first_m = extra * (base + 1) + b * rows_here;
        r = u - b * rows_here * n_blocks;
    }
    TileCoord c;
    c.m_blk = first_m + r % rows_here;
    const uint32_t n = r / rows_here;
    c.n_blk = (band & 1u) ? (n_blocks - 1u - n) : n;
    return c;
}

// Division of a 32-bit number by a divisor that is fixed for a whole launch, as a multiplication and two shifts
// (Granlund and Montgomery, "Division by invariant integers using multiplication"): the host computes the
// constants once, the kernels divide in a handful of cycles where the hardware's own division of two run-time
// values costs a couple of hundred -- which is what locating a tile used to cost the thread that issues the
// first loads of a kernel.
struct FastDiv {
    uint32_t divisor, mul, sh1, sh2;
};

inline FastDiv make_fast_div(uint32_t d) {
    FastDiv f;
    f.divisor = d < 1 ? 1u : d;
    uint32_t l = 0;
    while ((static_cast<uint64_t>(1) << l) < f.divisor) ++l;  // ceil(log2 d)
    f.mul = static_cast<uint32_t>(((static_cast<uint64_t>(1) << 32) * ((static_cast<uint64_t>(1) << l) - f.divisor)) / f.divisor + 1);
    f.sh1 = l < 1 ? l : 1u;
    f.sh2 = l > 0 ? l - 1 : 0u;
    return f;
}

B200_HD uint32_t fast_div(uint32_t n, const FastDiv &f) {
#if defined(__CUDA_ARCH__)
    const uint32_t t = __umulhi(f.mul, n);
#else
    const uint32_t t = static_cast<uint32_t>((static_cast<uint64_t>(f.mul) * n) >> 32);
#endif
    return (t + ((n - t) >> f.sh1)) >> f.sh2;
}

// tile_coord with everything that depends on the launch alone worked out beforehand.
struct Raster {
    uint32_t n_blocks, extra, base, tall_tiles;
    FastDiv tall_span, short_span, tall_rows, short_rows;  // (rows of a band) x n_blocks, and rows of a band
};

inline Raster make_raster(uint32_t m_blocks, uint32_t n_blocks, uint32_t group_m) {
    Raster r;
    if (group_m < 1) group_m = 1;
    if (m_blocks < 1) m_blocks = 1;
    if (n_blocks < 1) n_blocks = 1;
    const uint32_t bands = (m_blocks + group_m - 1) / group_m;
    r.n_blocks = n_blocks;
    r.base = m_blocks / bands;
    r.extra = m_blocks % bands;
    r.tall_tiles = r.extra * (r.base + 1) * n_blocks;
    r.tall_span = make_fast_div((r.base + 1) * n_blocks);
    r.short_span = make_fast_div((r.base < 1 ? 1u : r.base) * n_blocks);
    r.tall_rows = make_fast_div(r.base + 1);
    r.short_rows = make_fast_div(r.base < 1 ? 1u : r.base);
    return r;
}

// Same result as tile_coord(t, m_blocks, n_blocks, group_m) for the launch `r` was made for.
B200_HD TileCoord tile_coord_fast(uint32_t t, const Raster &r) {
    uint32_t band, first_m, rows_here, rem, n;
    if (t < r.tall_tiles) {
        rows_here = r.base + 1;
        band = fast_div(t, r.tall_span);
        first_m = band * rows_here;
        rem = t - band * rows_here * r.n_blocks;
        n = fast_div(rem, r.tall_rows);
    } else {
        rows_here = r.base;
        const uint32_t u = t - r.tall_tiles;
        const uint32_t b = fast_div(u, r.short_span);
        band = r.extra + b;
        first_m = r.extra * (r.base + 1) + b * rows_here;
        rem = u - b * rows_here * r.n_blocks;
        n = fast_div(rem, r.short_rows);
    }
    TileCoord c;
    c.m_blk = first_m + (rem - n * rows_here);
    c.n_blk = (band & 1u) ? (r.n_blocks - 1u - n) : n;
    return c;
}

// One contiguous piece of work: k-blocks [kb0, kb1) of output tile `tile`.
struct Segment {
    uint32_t tile;
    uint32_t kb0;
    uint32_t kb1;
};

// Stream-K: the `tiles * k_blocks` units (tile-major, k-minor) are cut into `parts` equal
// contiguous ranges; part p owns units [unit_begin(p), unit_begin(p+1)).
B200_HD uint64_t unit_begin(uint32_t part, uint32_t parts, uint64_t total_units) {
    return (static_cast<uint64_t>(part) * total_units) / parts;
}

// The part whose range contains unit u (largest p with unit_begin(p) <= u).
B200_HD uint32_t part_of_unit(uint64_t u, uint32_t parts, uint64_t total_units) {
    // unit_begin(p) <= u  <=>  p * total < (u + 1) * parts  <=>  p <= ceil((u+1)*parts/total) - 1
    uint64_t p = ((u + 1) * parts + total_units - 1) / total_units - 1;
    return static_cast<uint32_t>(p);
}

// Iterates the segments of one part in order.
struct SegmentWalker {
    uint64_t cur;
    uint64_t end;
    uint32_t k_blocks;

    B200_HD SegmentWalker(uint32_t part, uint32_t parts, uint32_t tiles, uint32_t k_blocks_) {
        const uint64_t total = static_cast<uint64_t>(tiles) * k_blocks_;
        cur = unit_begin(part, parts, total);
        end = unit_begin(part + 1, parts, total);
        k_blocks = k_blocks_;
    }

    B200_HD bool next(Segment &s) {
        if (cur >= end) return false;
        const uint32_t tile = static_cast<uint32_t>(cur / k_blocks);
        const uint32_t kb0 = static_cast<uint32_t>(cur - static_cast<uint64_t>(tile) * k_blocks);
        const uint64_t tile_end = (static_cast<uint64_t>(tile) + 1) * k_blocks;
        const uint64_t stop = tile_end < end ? tile_end : end;
        s.tile = tile;
        s.kb0 = kb0;
        s.kb1 = kb0 + static_cast<uint32_t>(stop - cur);
        cur = stop;
        return true;
    }
};

// Workspace slot a part writes its partial tile to: slot 0 for the first tile its range
// touches, slot 1 for any other (only the last tile of a range can also be partial).
B200_HD uint32_t partial_slot(uint32_t part, uint32_t parts, uint32_t tiles, uint32_t k_blocks, uint32_t tile) {
    const uint64_t total = static_cast<uint64_t>(tiles) * k_blocks;
    const uint32_t first_tile = static_cast<uint32_t>(unit_begin(part, parts, total) / k_blocks);
    return 2u * part + (tile == first_tile ? 0u : 1u);
}

}  // namespace b200
