// Device-side body of the weight-streaming matrix-vector product, shared by the stand-alone kernel
// (gemv.cu) and the persistent batch-1 decode kernel (decode.cu).
//
// Weights go HBM -> registers with 128-bit non-allocating loads (16 in flight per thread, 512 threads
// per SM). The activation vector of every matrix a block touches is prepared once in shared memory (int8
// high/low bytes of a 16-bit fixed-point value with one scale per 512 inputs, or fp16) and is shared by
// the four rows a warp works on. Work items are (4 rows x 2 KB slices of each row); one flat item list covers
// all matrices of a launch, so a launch has one prologue, one streaming loop and one epilogue. Per-item
// partial sums land in shared memory; a row-parallel epilogue sums the K slices in a fixed order, applies
// the row / tensor scale and the fused activation or residual, and stores fp16. Optionally a warp's first
// item of the NEXT phase is copied ahead of time into shared memory with cp.async; every variant of that
// measured slower than not doing it (the copies delay the loads of the next phase's input vector), so the
// persistent kernel leaves it off by default.
#pragma once
#include "gemv.cuh"

namespace ab {

constexpr int NT_CONS = GEMV_THREADS;

__device__ __forceinline__ void cons_sync() { __syncthreads(); }

// Activations written by other SMs earlier in the same kernel must not be served from a stale L1 line.
__device__ __forceinline__ uint4 ld_act16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
// Loads the compiler must issue where they are written (their consumers sit behind several barriers).
__device__ __forceinline__ float ld_early_f32(const float* p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_early_act_f16(const __half* p) {
    unsigned short v;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __half2float(__ushort_as_half(v));
}
// ---- tagged words (dataflow mode of the persistent kernel) -------------------------------------------------------
// word = fp16 bits | tag << 16. A reader spins until the tag is the one it expects: the load itself is the
// synchronisation (no barrier, no fence: every 32-bit word is written and read atomically and validates itself).
constexpr uint32_t TAG_SPIN_LIMIT = 1u << 21;
__device__ __forceinline__ uint32_t tag_of(uint32_t epoch, int stored) { return (epoch + (uint32_t)stored) & 0xffffu; }
__device__ __forceinline__ uint4 ld_relaxed_v4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_tagged(void* base, int idx, float v, uint32_t tag) {
    st_relaxed_u32(reinterpret_cast<uint32_t*>(base) + idx, (uint32_t)__half_as_ushort(__float2half_rn(v)) | (tag << 16));
}
// One tagged value; gives up (status bit, returns what is there) after a bounded number of tries.
__device__ __forceinline__ float ld_tagged1(const void* base, int idx, uint32_t tag) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(base) + idx;
    uint32_t w = ld_relaxed_u32(p), it = 0;
    while ((w >> 16) != tag) {
        if (++it > TAG_SPIN_LIMIT) {
            atomicOr(&g_device_status, DEV_WAIT_GEMV);
            break;
        }
        __nanosleep(TAG_POLL_NS);   // waiting blocks must not flood the L2 that the producers still need
        w = ld_relaxed_u32(p);
    }
    return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
}
// Eight consecutive tagged values (32-byte aligned) -> eight fp16 packed as a uint4.
__device__ __forceinline__ uint4 ld_tagged8(const void* base, int idx8, uint32_t tag) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(base) + 8 * (size_t)idx8;
    const uint32_t t = tag << 16;
    uint4 a, b;
    uint32_t it = 0;
    while (true) {
        a = ld_relaxed_v4(p);
        b = ld_relaxed_v4(p + 4);
        const uint32_t bad = ((a.x ^ t) | (a.y ^ t) | (a.z ^ t) | (a.w ^ t) | (b.x ^ t) | (b.y ^ t) | (b.z ^ t) | (b.w ^ t)) >> 16;
        if (!bad) break;
        if (++it > TAG_SPIN_LIMIT) {
            atomicOr(&g_device_status, DEV_WAIT_GEMV);
            break;
        }
        __nanosleep(TAG_POLL_NS);   // waiting blocks must not flood the L2 that the producers still need
    }
    return make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410), __byte_perm(b.x, b.y, 0x5410),
                      __byte_perm(b.z, b.w, 0x5410));
}
// Sixteen consecutive tagged values (64-byte aligned): all four loads in flight before the first is looked at.
__device__ __forceinline__ void ld_tagged16(const void* base, int idx16, uint32_t tag, uint4& lo, uint4& hi) {
    const uint32_t* p = reinterpret_cast<const uint32_t*>(base) + 16 * (size_t)idx16;
    const uint32_t t = tag << 16;
    uint4 a, b, c, d;
    uint32_t it = 0;
    while (true) {
        a = ld_relaxed_v4(p);
        b = ld_relaxed_v4(p + 4);
        c = ld_relaxed_v4(p + 8);
        d = ld_relaxed_v4(p + 12);
        const uint32_t bad = ((a.x ^ t) | (a.y ^ t) | (a.z ^ t) | (a.w ^ t) | (b.x ^ t) | (b.y ^ t) | (b.z ^ t) | (b.w ^ t) |
                              (c.x ^ t) | (c.y ^ t) | (c.z ^ t) | (c.w ^ t) | (d.x ^ t) | (d.y ^ t) | (d.z ^ t) | (d.w ^ t)) >> 16;
        if (!bad) break;
        if (++it > TAG_SPIN_LIMIT) {
            atomicOr(&g_device_status, DEV_WAIT_GEMV);
            break;
        }
        __nanosleep(TAG_POLL_NS);
    }
    lo = make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410), __byte_perm(b.x, b.y, 0x5410), __byte_perm(b.z, b.w, 0x5410));
    hi = make_uint4(__byte_perm(c.x, c.y, 0x5410), __byte_perm(c.z, c.w, 0x5410), __byte_perm(d.x, d.y, 0x5410), __byte_perm(d.z, d.w, 0x5410));
}
__device__ __forceinline__ void st_tagged8(void* base, int idx8, uint4 v, uint32_t tag) {
    uint32_t* p = reinterpret_cast<uint32_t*>(base) + 8 * (size_t)idx8;
    const uint32_t t = tag << 16, w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        st_relaxed_u32(p + 2 * e, (w[e] & 0xffffu) | t);
        st_relaxed_u32(p + 2 * e + 1, (w[e] >> 16) | t);
    }
}

// Start pulling a run of weights into L2 (no registers, no shared memory, nobody waits).
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// Weights are read exactly once: do not allocate them in L1.
__device__ __forceinline__ uint4 ld_w16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ---- shared-memory layout ------------------------------------------------------------------------
struct GemvLayout {
    size_t xn, dx, xq, sx, part, red, pref, total;
};
// Kn: length of the shared (normalised) input kept in smem, 0 if unused; with_dx: token-shift difference kept;
// xq_bytes: prepared inputs of all matrices one block can touch in a launch.
__host__ __device__ inline GemvLayout gemv_layout(int Kn, int with_dx, int xq_bytes) {
    GemvLayout L;
    const size_t Knp = ((size_t)Kn + 511) & ~(size_t)511;
    size_t off = 0;
    L.xn = off; off += Knp * 2;
    L.dx = off; off += with_dx ? Knp * 2 : 0;
    L.xq = off; off += (size_t)xq_bytes;
    L.sx = off; off += ((size_t)xq_bytes / 1024) * 4 + 32;
    L.part = off; off += (size_t)GEMV_PART_FLOATS * 4;
    L.red = off; off += 64 * 4;
    off = (off + 127) & ~(size_t)127;
    L.pref = off; off += (size_t)GEMV_WARPS * GEMV_ROWS * GEMV_SLICE_BYTES;   // one prefetched slice per warp
    L.total = off;
    return L;
}

struct GemvSmem {
    __half *xn, *dx;
    unsigned char* xq;
    float *sx, *part, *red;
    unsigned char* pref;
};
__device__ __forceinline__ GemvSmem gemv_smem(unsigned char* base, const GemvLayout& L) {
    GemvSmem m;
    m.xn = reinterpret_cast<__half*>(base + L.xn);
    m.dx = reinterpret_cast<__half*>(base + L.dx);
    m.xq = base + L.xq;
    m.sx = reinterpret_cast<float*>(base + L.sx);
    m.part = reinterpret_cast<float*>(base + L.part);
    m.red = reinterpret_cast<float*>(base + L.red);
    m.pref = base + L.pref;
    return m;
}

// ---- a block's share of a launch ---------------------------------------------------------------------
// Work is split between blocks in cost units (gemv_group_cost): block `bid` owns a contiguous cost range of
// the concatenated segments, i.e. a contiguous run of row groups in each segment it touches.
struct SegPlan {
    int lo, n_groups;        // first row group and number of row groups of this block in the segment
    int nks, row_bytes;      // K slices per row, bytes per row
    int chunk, npc;          // slices per work item (a run of consecutive slices of one row group), items per group
    int item_base, n_items;  // position of the segment's items in the block's flat item list
    int row_base;            // position of its rows in the block's flat row list
    int part_base;           // position of its partial sums
    int xq_off;              // byte offset of its prepared input in the xq area (sx offset = xq_off / 1024)
};
struct __align__(16) BlockPlan {
    SegPlan sp[GEMV_MAX_SEG];
    int n_items, n_rows, nseg, valid;
};

// 32-bit arithmetic on purpose (one thread computes this while the others run the prologue): costs are at
// most a few hundred thousand units and block counts a few hundred.
__host__ __device__ inline void compute_plan(const GemvParams& p, int bid, int nb, BlockPlan& bp) {
    unsigned total = 0;
    for (int s = 0; s < p.nseg; ++s)
        total += (unsigned)gemv_groups_of(p.seg[s].n_rows) * (unsigned)gemv_group_cost(p.seg[s].fmt, p.seg[s].K);
    const unsigned C0 = (unsigned)((unsigned long long)total * (unsigned)bid / (unsigned)nb);
    const unsigned C1 = (unsigned)((unsigned long long)total * (unsigned)(bid + 1) / (unsigned)nb);
    unsigned base = 0;
    int items = 0, rows = 0, part = 0, xq = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const GemvSeg& sg = p.seg[s];
        const unsigned n = (unsigned)gemv_groups_of(sg.n_rows), unit = (unsigned)gemv_group_cost(sg.fmt, sg.K);
        unsigned l = C0 <= base ? 0u : (C0 - base + unit - 1) / unit;
        unsigned h = C1 <= base ? 0u : (C1 - base + unit - 1) / unit;
        if (l > n) l = n;
        if (h > n) h = n;
        SegPlan& q = bp.sp[s];
        q.lo = (int)l;
        q.n_groups = (int)(h - l);
        q.nks = gemv_slices(sg.fmt, sg.K);
        q.row_bytes = gemv_row_bytes(sg.fmt, sg.K);
        // longer items (fewer reductions and partial sums) as long as every warp still gets about two of them
        int chunk = 1;
        while (chunk * 2 <= q.nks && q.nks % (chunk * 2) == 0 && q.n_groups * (q.nks / (chunk * 2)) >= 2 * GEMV_WARPS)
            chunk *= 2;
        q.chunk = chunk;
        q.npc = q.nks / chunk;
        q.item_base = items;
        q.n_items = q.n_groups * q.npc;
        q.row_base = rows;
        q.part_base = part;
        q.xq_off = xq;
        items += q.n_items;
        rows += q.n_groups * GEMV_ROWS;
        part += q.n_groups * GEMV_ROWS * q.npc;
        if (q.n_groups > 0) xq += gemv_xq_bytes(sg.K);
        base += n * unit;
    }
    bp.n_items = items;
    bp.n_rows = rows;
    bp.nseg = p.nseg;
    bp.valid = 1;
}

// Plan that gives block `bid` the rows [bid * rows_per_block, (bid + 1) * rows_per_block) of EVERY segment (and
// nothing to blocks past the last row): used when a later step of the same block consumes exactly those
// rows, e.g. the per-head adapter up-projections that feed the head's own WKV step.
__host__ __device__ inline void compute_plan_rows(const GemvParams& p, int bid, int rows_per_block, BlockPlan& bp) {
    int items = 0, rows = 0, part = 0, xq = 0;
    for (int s = 0; s < p.nseg; ++s) {
        const GemvSeg& sg = p.seg[s];
        const int n = gemv_groups_of(sg.n_rows), gpb = rows_per_block / GEMV_ROWS;
        int l = bid * gpb, h = l + gpb;
        if (l > n) l = n;
        if (h > n) h = n;
        SegPlan& q = bp.sp[s];
        q.lo = l;
        q.n_groups = h - l;
        q.nks = gemv_slices(sg.fmt, sg.K);
        q.row_bytes = gemv_row_bytes(sg.fmt, sg.K);
        q.chunk = q.nks;
        q.npc = 1;
        q.item_base = items;
        q.n_items = q.n_groups * q.npc;
        q.row_base = rows;
        q.part_base = part;
        q.xq_off = xq;
        items += q.n_items;
        rows += q.n_groups * GEMV_ROWS;
        part += q.n_groups * GEMV_ROWS * q.npc;
        if (q.n_groups > 0) xq += gemv_xq_bytes(sg.K);
    }
    bp.n_items = items;
    bp.n_rows = rows;
    bp.nseg = p.nseg;
    bp.valid = 1;
}

// Plan of the r/k/v + adapter phase of the persistent kernel in dataflow mode. Segments 0..2 are the r, k, v matrices,
// the rest the adapter down-projections. Blocks 2h and 2h + 1 compute the 64 rows of head h of each of r, k, v (48 row
// groups in the order r, k, v: the first `split` go to block 2h, which also runs the head afterwards and holds its
// up-projection weights, the others to block 2h + 1); blocks 2H .. nb - 1 share the adapter rows by cost.
__host__ inline void compute_plan_heads(const GemvParams& p, int bid, int nb, int H, int split, BlockPlan& bp) {
    int items = 0, rows = 0, part = 0, xq = 0;
    auto fill = [&](int s, int lo, int n_groups) {
        const GemvSeg& sg = p.seg[s];
        SegPlan& q = bp.sp[s];
        q.lo = lo;
        q.n_groups = n_groups;
        q.nks = gemv_slices(sg.fmt, sg.K);
        q.row_bytes = gemv_row_bytes(sg.fmt, sg.K);
        int chunk = 1;
        while (chunk * 2 <= q.nks && q.nks % (chunk * 2) == 0 && q.n_groups * (q.nks / (chunk * 2)) >= 2 * GEMV_WARPS) chunk *= 2;
        q.chunk = chunk;
        q.npc = q.nks / chunk;
        q.item_base = items;
        q.n_items = q.n_groups * q.npc;
        q.row_base = rows;
        q.part_base = part;
        q.xq_off = xq;
        items += q.n_items;
        rows += q.n_groups * GEMV_ROWS;
        part += q.n_groups * GEMV_ROWS * q.npc;
        if (q.n_groups > 0) xq += gemv_xq_bytes(sg.K);
    };
    const int gph = HEAD / GEMV_ROWS;   // row groups per head and matrix
    if (bid < 2 * H) {
        // the head's 3 * gph row groups in the order r, k, v: block 2h takes the first `split`, block 2h + 1 the rest, so
        // that each of them prepares the inputs of two matrices at most
        const int h = bid >> 1, odd = bid & 1;
        const int g0 = odd ? split : 0, g1 = odd ? 3 * gph : split;
        for (int s = 0; s < p.nseg; ++s) {
            int lo = 0, n = 0;
            if (s < 3) {
                const int a = g0 > s * gph ? g0 : s * gph, b = g1 < (s + 1) * gph ? g1 : (s + 1) * gph;
                if (b > a) { lo = h * gph + a - s * gph; n = b - a; }
            }
            fill(s, lo, n);
        }
    } else {
        const int b = bid - 2 * H, nd = nb - 2 * H;
        unsigned total = 0;
        for (int s = 3; s < p.nseg; ++s)
            total += (unsigned)gemv_groups_of(p.seg[s].n_rows) * (unsigned)gemv_group_cost(p.seg[s].fmt, p.seg[s].K);
        const unsigned C0 = (unsigned)((unsigned long long)total * (unsigned)b / (unsigned)nd);
        const unsigned C1 = (unsigned)((unsigned long long)total * (unsigned)(b + 1) / (unsigned)nd);
        unsigned base = 0;
        for (int s = 0; s < p.nseg; ++s) {
            if (s < 3) { fill(s, 0, 0); continue; }
            const unsigned n = (unsigned)gemv_groups_of(p.seg[s].n_rows), unit = (unsigned)gemv_group_cost(p.seg[s].fmt, p.seg[s].K);
            unsigned l = C0 <= base ? 0u : (C0 - base + unit - 1) / unit;
            unsigned hgh = C1 <= base ? 0u : (C1 - base + unit - 1) / unit;
            if (l > n) l = n;
            if (hgh > n) hgh = n;
            fill(s, (int)l, (int)(hgh - l));
            base += n * unit;
        }
    }
    bp.n_items = items;
    bp.n_rows = rows;
    bp.nseg = p.nseg;
    bp.valid = 1;
}

// Ask for bytes [skip, skip + bytes) of a block's share of a launch (its rows of each segment, in plan order: the order
// its warps consume them in) to be moved HBM -> L2. Called by one thread.
__device__ __forceinline__ void prefetch_share(const GemvParams& q, const BlockPlan& bp, int skip, int bytes) {
    for (int s = 0; s < q.nseg && bytes > 0; ++s) {
        const SegPlan& sp = bp.sp[s];
        if (sp.n_groups <= 0) continue;
        const int row0 = sp.lo * GEMV_ROWS;
        const int total = min(sp.n_groups * GEMV_ROWS, q.seg[s].n_rows - row0) * sp.row_bytes;
        if (skip >= total) {
            skip -= total;
            continue;
        }
        const int n = min(total - skip, bytes) & ~15;
        if (n > 0) prefetch_l2((const unsigned char*)q.seg[s].w + (size_t)row0 * sp.row_bytes + skip, (uint32_t)n);
        bytes -= n;
        skip = 0;
    }
}

// ---- work items ------------------------------------------------------------------------------------
// In bytes every format looks the same: an item is GEMV_ROWS rows x 1024 bytes of each row starting at byte
// `sb`; lane l reads bytes [sb + u*512 + l*16, +16) of each row for u = 0, 1.
struct Item {
    const unsigned char* w0;   // first row of the group
    const unsigned char* s0;   // its NVFP4 block scales (else null)
    int row_bytes, rows, sb;   // sb: first byte of the item in each row
    int n_slices;              // consecutive 1 KB slices in this item
    int seg, pidx;             // segment; index of the item's first partial sum (+ lane * npc per row)
};
struct ItemBuf {
    uint4 w[GEMV_SWEEPS][GEMV_ROWS];
    uint32_t sc[GEMV_SWEEPS / 2][GEMV_ROWS];    // NVFP4: two e4m3 scales per sweep, even sweep in the low half
};

// Item `i` of the block's flat list.
__device__ __forceinline__ Item make_item(const GemvParams& p, const BlockPlan& bp, int i) {
    int s = 0;
    while (s + 1 < bp.nseg && i >= bp.sp[s].item_base + bp.sp[s].n_items) ++s;
    const SegPlan& q = bp.sp[s];
    const GemvSeg& sg = p.seg[s];
    const int it = i - q.item_base;
    const int gl = it / q.npc, sl = it - gl * q.npc;
    const int row0 = (q.lo + gl) * GEMV_ROWS;
    Item t;
    t.row_bytes = q.row_bytes;
    t.rows = min(GEMV_ROWS, sg.n_rows - row0);
    t.sb = sl * q.chunk * GEMV_SLICE_BYTES;
    t.n_slices = q.chunk;
    t.w0 = (const unsigned char*)sg.w + (size_t)row0 * q.row_bytes;
    t.s0 = sg.fmt == FMT_FP4 ? (const unsigned char*)sg.scale + (size_t)row0 * (sg.K / 16) : nullptr;
    t.seg = s;
    t.pidx = q.part_base + gl * GEMV_ROWS * q.npc + sl;
    return t;
}

// Issue the 16 (+ scale) loads of slice `slice` of an item; nothing waits for them here.
// FULL: all four rows exist and the slice lies inside the row, so no load is predicated.
template <bool FULL>
__device__ __forceinline__ void load_item(const Item& t, int slice, int lane, ItemBuf& b) {
    const int o = t.sb + slice * GEMV_SLICE_BYTES + lane * 16;
    const unsigned char* p0 = t.w0 + o;
#pragma unroll
    for (int r = 0; r < GEMV_ROWS; ++r) {
        const unsigned char* pr = p0 + (size_t)r * t.row_bytes;
#pragma unroll
        for (int u = 0; u < GEMV_SWEEPS; ++u) {
            if ((FULL || (o + u * 512 < t.row_bytes && r < t.rows)) && AB_BC(o + u * 512 + 16 <= t.row_bytes && r < t.rows))
                b.w[u][r] = ld_w16(pr + u * 512);
            else b.w[u][r] = make_uint4(0, 0, 0, 0);
        }
    }
    if (t.s0) {
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
            for (int u2 = 0; u2 < GEMV_SWEEPS / 2; ++u2) {
                uint32_t v = 0;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int oo = o + (2 * u2 + h) * 512;
                    if (FULL || (oo < t.row_bytes && r < t.rows))
                        v |= (uint32_t)(*reinterpret_cast<const unsigned short*>(t.s0 + (size_t)r * (t.row_bytes / 8) + oo / 8)) << (16 * h);
                }
                b.sc[u2][r] = v;
            }
    }
}
// Copy slice 0 of an item into the warp's slot of shared memory without waiting (cp.async, zero fill where invalid).
__device__ __forceinline__ void prefetch_item(const Item& t, int lane, unsigned char* slot) {
#pragma unroll
    for (int u = 0; u < GEMV_SWEEPS; ++u) {
        const int o = t.sb + u * 512 + lane * 16;
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r) {
            const bool ok = o < t.row_bytes && r < t.rows;
            const unsigned char* src = ok ? t.w0 + (size_t)r * t.row_bytes + o : t.w0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(slot + (u * GEMV_ROWS + r) * 512 + lane * 16)),
                         "l"(src), "r"(ok ? 16 : 0)
                         : "memory");
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
// Collect a prefetched slice from the warp's slot (each lane reads back exactly what it copied).
__device__ __forceinline__ void take_prefetched(const Item& t, int lane, const unsigned char* slot, ItemBuf& b) {
    asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
    for (int u = 0; u < GEMV_SWEEPS; ++u)
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r)
            b.w[u][r] = *reinterpret_cast<const uint4*>(slot + (u * GEMV_ROWS + r) * 512 + lane * 16);
    if (t.s0) {
        const int o = t.sb + lane * 16;
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
            for (int u2 = 0; u2 < GEMV_SWEEPS / 2; ++u2) {
                uint32_t v = 0;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int oo = o + (2 * u2 + h) * 512;
                    if (oo < t.row_bytes && r < t.rows)
                        v |= (uint32_t)(*reinterpret_cast<const unsigned short*>(t.s0 + (size_t)r * (t.row_bytes / 8) + oo / 8)) << (16 * h);
                }
                b.sc[u2][r] = v;
            }
    }
}

// acc[r] += this lane's part of (row r, slice `slice` of the item). xq / sx: the segment's prepared input.
template <int FMT, bool FULL>
__device__ __forceinline__ void compute_item(const Item& t, int slice, const ItemBuf& b, const unsigned char* xq, int Kp,
                                             const float* sx, int lane, float* acc) {
#pragma unroll
    for (int u = 0; u < GEMV_SWEEPS; ++u) {
        const int o = t.sb + slice * GEMV_SLICE_BYTES + u * 512 + lane * 16;
        if (FULL || o < t.row_bytes) {
            if (FMT == FMT_I8) {
                const uint4 a = *reinterpret_cast<const uint4*>(xq + o);
                const uint4 c = *reinterpret_cast<const uint4*>(xq + Kp + o);
                const float scl = sx[o >> 9];
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; ++r) {
                    const uint4 w = b.w[u][r];
                    int ah = __dp4a((int)w.x, (int)a.x, 0);
                    int al = __dp4a((int)w.x, (int)c.x, 0);
                    ah = __dp4a((int)w.y, (int)a.y, ah);
                    al = __dp4a((int)w.y, (int)c.y, al);
                    ah = __dp4a((int)w.z, (int)a.z, ah);
                    al = __dp4a((int)w.z, (int)c.z, al);
                    ah = __dp4a((int)w.w, (int)a.w, ah);
                    al = __dp4a((int)w.w, (int)c.w, al);
                    acc[r] = fmaf((float)(ah * 256 + al), scl, acc[r]);
                }
            } else if (FMT == FMT_F16) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xq + o);   // 8 inputs
                const __half2* x2 = reinterpret_cast<const __half2*>(&xv);
                float2 xf[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) xf[e] = __half22float2(x2[e]);
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; ++r) {
                    const __half2* w2 = reinterpret_cast<const __half2*>(&b.w[u][r]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 wf = __half22float2(w2[e]);
                        acc[r] = fmaf(wf.x, xf[e].x, acc[r]);
                        acc[r] = fmaf(wf.y, xf[e].y, acc[r]);
                    }
                }
            } else {  // NVFP4: 16 bytes = 32 inputs = two scale blocks
                uint4 xv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) xv[e] = *reinterpret_cast<const uint4*>(xq + (size_t)o * 4 + e * 16);
                const __half2* x2 = reinterpret_cast<const __half2*>(xv);
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; ++r) {
                    const float2 scf = __half22float2(e4m3x2_to_half2((b.sc[u >> 1][r] >> (16 * (u & 1))) & 0xffffu));
                    const uint4 w = b.w[u][r];
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int bl = 0; bl < 2; ++bl) {
                        __half2 h = __floats2half2_rn(0.f, 0.f);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const uint32_t byte = (ww[bl * 2 + (e >> 2)] >> (8 * (e & 3))) & 0xffu;
                            h = __hfma2(e2m1x2_to_half2(byte), x2[bl * 8 + e], h);
                        }
                        const float2 hf = __half22float2(h);
                        acc[r] = fmaf(hf.x + hf.y, bl ? scf.y : scf.x, acc[r]);
                    }
                }
            }
        }
    }
}

// All slices of an item whose first slice is already in `cb`.
template <int FMT, bool FULL>
__device__ __forceinline__ void run_item(const Item& t, ItemBuf& cb, const unsigned char* xq, int Kp, const float* sx,
                                         int lane, float* acc) {
    for (int sl = 0; sl < t.n_slices; ++sl) {
        compute_item<FMT, FULL>(t, sl, cb, xq, Kp, sx, lane, acc);
        if (sl + 1 < t.n_slices) load_item<FULL>(t, sl + 1, lane, cb);
    }
}
__device__ __forceinline__ bool item_full(const Item& t) {
    return t.rows == GEMV_ROWS && (t.row_bytes & (GEMV_SLICE_BYTES - 1)) == 0;
}

// Block-wide sums of two values with one pair of barriers.
__device__ __forceinline__ float2 cons_block_sum2(float a, float b, float* red, int tid) {
    a = warp_sum(a);
    b = warp_sum(b);
    cons_sync();
    if ((tid & 31) == 0) {
        red[tid >> 5] = a;
        red[32 + (tid >> 5)] = b;
    }
    cons_sync();
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int i = 0; i < GEMV_WARPS; ++i) {
        ta += red[i];
        tb += red[32 + i];
    }
    return make_float2(ta, tb);
}

// Prepare 512 inputs (block `kb`) of one segment's input in shared memory in the form its rows consume: one warp, 16
// elements per lane.
__device__ __forceinline__ void prep_x_block(const GemvSeg& sg, const GemvSmem& m, int xq_off, int kb, int lane, uint32_t epoch) {
    const int K = sg.K, Kp = (K + 511) & ~511;
    unsigned char* xq = m.xq + xq_off;
    float* sx = m.sx + xq_off / 1024;
    {
        const int c0 = kb * 32;
        const int c = c0 + lane;
        const bool in = c * 16 < K;
        float v[16];
        if (in) {
            uint4 a0, a1;
            if (sg.x && sg.tag_x) {
                ld_tagged16(sg.x, c, tag_of(epoch, sg.tag_x), a0, a1);
            } else if (sg.x) {
                a0 = ld_act16(reinterpret_cast<const uint4*>(sg.x) + 2 * c);
                a1 = ld_act16(reinterpret_cast<const uint4*>(sg.x) + 2 * c + 1);
            } else {
                a0 = reinterpret_cast<const uint4*>(m.xn)[2 * c];
                a1 = reinterpret_cast<const uint4*>(m.xn)[2 * c + 1];
            }
            const __half2* h0 = reinterpret_cast<const __half2*>(&a0);
            const __half2* h1 = reinterpret_cast<const __half2*>(&a1);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f0 = __half22float2(h0[e]), f1 = __half22float2(h1[e]);
                v[2 * e] = f0.x;
                v[2 * e + 1] = f0.y;
                v[8 + 2 * e] = f1.x;
                v[9 + 2 * e] = f1.y;
            }
            if (sg.mix) {
                const uint4 d0 = reinterpret_cast<const uint4*>(m.dx)[2 * c], d1 = reinterpret_cast<const uint4*>(m.dx)[2 * c + 1];
                const uint4 m0 = reinterpret_cast<const uint4*>(sg.mix)[2 * c], m1 = reinterpret_cast<const uint4*>(sg.mix)[2 * c + 1];
                const __half2* dd[2] = {reinterpret_cast<const __half2*>(&d0), reinterpret_cast<const __half2*>(&d1)};
                const __half2* mm[2] = {reinterpret_cast<const __half2*>(&m0), reinterpret_cast<const __half2*>(&m1)};
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 df = __half22float2(dd[hh][e]), mf = __half22float2(mm[hh][e]);
                        v[8 * hh + 2 * e] = rh(v[8 * hh + 2 * e] + rh(df.x * mf.x));
                        v[8 * hh + 2 * e + 1] = rh(v[8 * hh + 2 * e + 1] + rh(df.y * mf.y));
                    }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = 0.f;
        }
        if (sg.fmt != FMT_I8) {
            if (in) {
                __half2 h[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                if (AB_BC(c * 32 + 32 <= 2 * Kp)) {
                    reinterpret_cast<uint4*>(xq)[c * 2] = *reinterpret_cast<uint4*>(&h[0]);
                    reinterpret_cast<uint4*>(xq)[c * 2 + 1] = *reinterpret_cast<uint4*>(&h[4]);
                }
            }
        } else {
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                if (sg.col_scale && in) v[e] *= sg.col_scale[c * 16 + e];
                amax = fmaxf(amax, fabsf(v[e]));
            }
            amax = warp_max(amax);  // one scale per 512 inputs = the 32 chunks of this warp pass
            // X = 256 * h + l with h, l both signed bytes: |X| <= 127 * 256 + 127
            const float inv = amax > 0.f ? 32639.0f / amax : 0.f;
            uint32_t hw[4], lw[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t hh = 0, ll = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int X = __float2int_rn(v[q * 4 + e] * inv);
                    const int hi8 = (X + 128) >> 8;
                    hh |= (uint32_t)(hi8 & 0xff) << (8 * e);
                    ll |= (uint32_t)((X - (hi8 << 8)) & 0xff) << (8 * e);
                }
                hw[q] = hh;
                lw[q] = ll;
            }
            if (AB_BC(c * 16 + 16 <= Kp)) {
                reinterpret_cast<uint4*>(xq)[c] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                reinterpret_cast<uint4*>(xq + Kp)[c] = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            }
            if (lane == 0) sx[c0 / 32] = amax / 32639.0f;
        }
    }
}

// ---- one launch / phase ----------------------------------------------------------------------------
// Called by all threads of a block.
//   bp      : this block's plan for p (shared memory, already computed and visible to all threads)
//   pre_phase : launch phase whose item `warp` sits in the warp's prefetch slot, or -1
//   np, nbp : the next matrix-vector launch and this block's plan for it (or null): each warp copies its
//             first item of that launch into its slot when it runs out of items here
struct NoHook {
    __device__ __forceinline__ void operator()() const {}
};
// after_prep: called by every thread once the block's inputs are prepared, right before the weight stream starts (work
// that may share the memory pipe with the stream but must not sit in front of the input vector's loads).
template <class AfterPrep = NoHook>
__device__ __forceinline__ void gemv_consume(const GemvParams& p, const BlockPlan& bp, const GemvSmem& m, int tid,
                                             int bid, int phase_idx, int& pre_phase, const GemvParams* np,
                                             const BlockPlan* nbp, int next_phase_idx, unsigned long long* tl = nullptr,
                                             int early = 0, AfterPrep after_prep = AfterPrep(), uint32_t epoch = 0,
                                             int pf_skip = 0, int pf_bytes = 0) {
    auto stamp = [&](int k) {
        if (tl && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            tl[k] = t;
        }
    };
    const int warp = tid >> 5, lane = tid & 31;
    __half* xn = m.xn;
    __half* dx = m.dx;
    // `early`: the first slice of the warp's first item is requested (cp.async into the warp's slot) right behind
    // the input vector's loads, so that it is there when the inputs have been prepared. Asked for any earlier, the
    // weight traffic would sit in front of the input loads in the memory pipeline and delay them.
    bool early_issued = false;
    auto issue_early = [&]() {
        if (early && !early_issued && pre_phase != phase_idx && warp < bp.n_items) {
            prefetch_item(make_item(p, bp, warp), lane, m.pref + warp * (GEMV_ROWS * GEMV_SLICE_BYTES));
            early_issued = true;
        }
    };

    // dataflow mode: the input is waited for below (tagged words); the first weight slice travels in the meantime
    if (epoch && early == 1) issue_early();

    if (p.copy_src && bid == 0)
        for (int i = tid; i < p.copy_n / 8; i += NT_CONS)
            reinterpret_cast<uint4*>(p.copy_dst)[i] = ld_act16(reinterpret_cast<const uint4*>(p.copy_src) + i);

    // ---- epilogue operands of this thread's output row: loaded now, used at the end
    int e_seg = -1, e_row = 0;
    float e_scale = 1.f, e_resid = 0.f;
    if (tid < bp.n_rows) {
        int s = 0;
        while (s + 1 < bp.nseg && tid >= bp.sp[s].row_base + bp.sp[s].n_groups * GEMV_ROWS) ++s;
        const GemvSeg& sg = p.seg[s];
        const int row = bp.sp[s].lo * GEMV_ROWS + (tid - bp.sp[s].row_base);
        if (row < sg.n_rows) {
            e_seg = s;
            e_row = row;
            e_scale = sg.fmt == FMT_I8 ? ld_early_f32(reinterpret_cast<const float*>(sg.scale) + row) : sg.tscale;
            if (sg.epi == EPI_RESID)
                e_resid = sg.tag_resid ? ld_tagged1(sg.resid, row, tag_of(epoch, sg.tag_resid)) : ld_early_act_f16(sg.resid + row);
        }
    }

    // ---- shared input vector, optional layer norm, token-shift difference
    const bool shared_in = p.emb || p.x;
    if (shared_in) {
        const int K = p.K;
        const __half* xin = p.x;
        if (p.emb) {
            int tok = __ldcg(p.token);
            if ((unsigned)tok >= (unsigned)p.emb_rows) {   // never index past the table: clamp and tell the host
                tok = tok < 0 ? 0 : p.emb_rows - 1;
                if (tid == 0 && bid == 0) atomicOr(&g_device_status, DEV_BAD_TOKEN);
            }
            xin = p.emb + (size_t)tok * K;
        }
        bool any_mix = false;
        for (int s = 0; s < p.nseg; ++s) any_mix |= p.seg[s].mix != nullptr;
        // One pass when K / 8 <= threads (every thread keeps its 8 inputs, weights, bias and previous inputs in
        // registers: all four loads are in flight together); longer inputs loop over the same code.
        const bool ln = p.ln_w != nullptr;
        float lsum = 0.f, lsq = 0.f;
        for (int i0 = 0; i0 < K / 8; i0 += NT_CONS) {
            const int i = i0 + tid;
            const bool in = i < K / 8;
            uint4 v = make_uint4(0, 0, 0, 0), wv = v, bv = v, pv = v;
            if (in) {
                v = (p.tag_in && !p.emb) ? ld_tagged8(xin, i, tag_of(epoch, p.tag_in)) : ld_act16(reinterpret_cast<const uint4*>(xin) + i);
                if (ln) {
                    wv = reinterpret_cast<const uint4*>(p.ln_w)[i];
                    bv = reinterpret_cast<const uint4*>(p.ln_b)[i];
                }
                if (any_mix) pv = ld_act16(reinterpret_cast<const uint4*>(p.x_prev) + i);
                if (p.x_copy && bid == 0) {
                    if (p.tag_in) st_tagged8(p.x_copy, i, v, tag_of(epoch, p.tag_in));
                    else reinterpret_cast<uint4*>(p.x_copy)[i] = v;
                }
            }
            issue_early();
            const __half2* h = reinterpret_cast<const __half2*>(&v);
            if (K / 8 <= NT_CONS) {
                // single pass: statistics over the whole vector are available after one block reduction
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h[e]);
                    lsum += f.x + f.y;
                    lsq = fmaf(f.x, f.x, fmaf(f.y, f.y, lsq));
                }
                uint4 o = v;
                if (ln) {
                    const float2 st = cons_block_sum2(lsum, lsq, m.red, tid);
                    const float mean = st.x / (float)K;
                    const float rstd = rsqrtf(fmaxf(st.y / (float)K - mean * mean, 0.f) + 1e-5f);
                    const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
                    const __half2* b2 = reinterpret_cast<const __half2*>(&bv);
                    __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(h[e]), wf = __half22float2(w2[e]), bf = __half22float2(b2[e]);
                        o2[e] = __floats2half2_rn((f.x - mean) * rstd * wf.x + bf.x, (f.y - mean) * rstd * wf.y + bf.y);
                    }
                }
                if (in) {
                    reinterpret_cast<uint4*>(xn)[i] = o;
                    if (ln && p.ln_out && bid == 0) reinterpret_cast<uint4*>(p.ln_out)[i] = o;
                    if (any_mix) {
                        const __half2* o2 = reinterpret_cast<const __half2*>(&o);
                        const __half2* q2 = reinterpret_cast<const __half2*>(&pv);
                        uint4 d;
                        __half2* d2 = reinterpret_cast<__half2*>(&d);
#pragma unroll
                        for (int e = 0; e < 4; ++e) d2[e] = __hsub2(q2[e], o2[e]);
                        reinterpret_cast<uint4*>(dx)[i] = d;
                    }
                }
            } else {
                // long shared inputs (no launch of the decode path has one with a layer norm): stage and sum
                if (in) {
                    reinterpret_cast<uint4*>(xn)[i] = v;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(h[e]);
                        lsum += f.x + f.y;
                        lsq = fmaf(f.x, f.x, fmaf(f.y, f.y, lsq));
                    }
                }
            }
        }
        if (K / 8 > NT_CONS) {
            float mean = 0.f, rstd = 1.f;
            if (ln) {
                const float2 st = cons_block_sum2(lsum, lsq, m.red, tid);
                mean = st.x / (float)K;
                rstd = rsqrtf(fmaxf(st.y / (float)K - mean * mean, 0.f) + 1e-5f);
            }
            for (int i = tid; i < K / 8; i += NT_CONS) {   // the same thread staged xn[i]: no barrier needed
                uint4 o = reinterpret_cast<const uint4*>(xn)[i];
                if (ln) {
                    const uint4 wv = reinterpret_cast<const uint4*>(p.ln_w)[i];
                    const uint4 bv = reinterpret_cast<const uint4*>(p.ln_b)[i];
                    const __half2* w2 = reinterpret_cast<const __half2*>(&wv);
                    const __half2* b2 = reinterpret_cast<const __half2*>(&bv);
                    __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(o2[e]), wf = __half22float2(w2[e]), bf = __half22float2(b2[e]);
                        o2[e] = __floats2half2_rn((f.x - mean) * rstd * wf.x + bf.x, (f.y - mean) * rstd * wf.y + bf.y);
                    }
                    reinterpret_cast<uint4*>(xn)[i] = o;
                    if (p.ln_out && bid == 0) reinterpret_cast<uint4*>(p.ln_out)[i] = o;
                }
                if (any_mix) {
                    const uint4 pv = ld_act16(reinterpret_cast<const uint4*>(p.x_prev) + i);
                    const __half2* o2 = reinterpret_cast<const __half2*>(&o);
                    const __half2* q2 = reinterpret_cast<const __half2*>(&pv);
                    uint4 d;
                    __half2* d2 = reinterpret_cast<__half2*>(&d);
#pragma unroll
                    for (int e = 0; e < 4; ++e) d2[e] = __hsub2(q2[e], o2[e]);
                    reinterpret_cast<uint4*>(dx)[i] = d;
                }
            }
        }
        cons_sync();
    }
    stamp(0);
    // every producer of the inputs is done, so no block streams weights any more: the memory system idles while the
    // inputs are prepared. More of this block's share moves into L2 in that time.
    if (pf_bytes > 0 && tid == 32) prefetch_share(p, bp, pf_skip, pf_bytes);
    issue_early();

    // ---- prepared inputs of every segment this block touches
    {   // warp tasks = (segment the block touches, 512-input block of its input), dealt round-robin to all warps
        int t = warp;   // this warp's next task, counted from the first block of the current segment
        for (int s = 0; s < bp.nseg; ++s) {
            if (bp.sp[s].n_groups <= 0) continue;
            const int nb_k = (p.seg[s].K + 511) >> 9;
            for (; t < nb_k; t += GEMV_WARPS) prep_x_block(p.seg[s], m, bp.sp[s].xq_off, t, lane, epoch);
            t -= nb_k;
        }
    }
    cons_sync();
    stamp(1);
    after_prep();

    // ---- stream the block's items: warp w takes items w, w + 32, ...
    if (warp < bp.n_items) {
        unsigned char* slot = m.pref + warp * (GEMV_ROWS * GEMV_SLICE_BYTES);
        Item cur = make_item(p, bp, warp);
        ItemBuf cb;
        if (pre_phase == phase_idx || early_issued) take_prefetched(cur, lane, slot, cb);   // the slot holds slice 0 of item `warp`
        else if (item_full(cur)) load_item<true>(cur, 0, lane, cb);
        else load_item<false>(cur, 0, lane, cb);
        int i = warp;
        while (true) {
            float acc[GEMV_ROWS];
#pragma unroll
            for (int r = 0; r < GEMV_ROWS; ++r) acc[r] = 0.f;
            const GemvSeg& sg = p.seg[cur.seg];
            const SegPlan& q = bp.sp[cur.seg];
            const unsigned char* xq = m.xq + q.xq_off;
            const float* sx = m.sx + q.xq_off / 1024;
            const int Kp = (sg.K + 511) & ~511, fmt = sg.fmt;
            const bool full = item_full(cur);
            if (fmt == FMT_I8) {
                if (full) run_item<FMT_I8, true>(cur, cb, xq, Kp, sx, lane, acc);
                else run_item<FMT_I8, false>(cur, cb, xq, Kp, sx, lane, acc);
            } else if (fmt == FMT_F16) {
                if (full) run_item<FMT_F16, true>(cur, cb, xq, Kp, sx, lane, acc);
                else run_item<FMT_F16, false>(cur, cb, xq, Kp, sx, lane, acc);
            } else {
                if (full) run_item<FMT_FP4, true>(cur, cb, xq, Kp, sx, lane, acc);
                else run_item<FMT_FP4, false>(cur, cb, xq, Kp, sx, lane, acc);
            }
            const int pidx = cur.pidx, npc = q.npc;
            i += GEMV_WARPS;
            const bool more = i < bp.n_items;
            if (more) {   // issue the next item's first loads before the reduction of this one
                cur = make_item(p, bp, i);
                if (item_full(cur)) load_item<true>(cur, 0, lane, cb);
                else load_item<false>(cur, 0, lane, cb);
            }
#pragma unroll
            for (int r = 0; r < GEMV_ROWS; ++r) acc[r] = warp_sum(acc[r]);
            if (lane < GEMV_ROWS) {
                float val = 0.f;
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; ++r)
                    if (r == lane) val = acc[r];
                if (AB_BC(pidx + lane * npc >= 0 && pidx + lane * npc < GEMV_PART_FLOATS)) m.part[pidx + lane * npc] = val;
            }
            if (!more) break;
        }
    }
    stamp(2);
    pre_phase = -1;
    // ---- the warp's first item of the next launch starts its way into shared memory now
    if (np && nbp && warp < nbp->n_items) {
        const Item t = make_item(*np, *nbp, warp);
        prefetch_item(t, lane, m.pref + warp * (GEMV_ROWS * GEMV_SLICE_BYTES));
        pre_phase = next_phase_idx;
    }
    cons_sync();
    stamp(3);

    // ---- epilogue: one thread per output row of the block
    if (e_seg >= 0) {
        const GemvSeg& sg = p.seg[e_seg];
        const SegPlan& q = bp.sp[e_seg];
        const int rl = tid - q.row_base;
        float val = 0.f;
        for (int sl = 0; sl < q.npc; ++sl)
            if (AB_BC(q.part_base + rl * q.npc + sl < GEMV_PART_FLOATS)) val += m.part[q.part_base + rl * q.npc + sl];
        float o = rh(val * e_scale);
        switch (sg.epi) {
            case EPI_TANH: o = tanhf(o); break;
            case EPI_SIGMOID: o = sigmoidf_(o); break;
            case EPI_RELU2: o = fmaxf(o, 0.f); o = o * o; break;
            case EPI_RESID: o = e_resid + o; break;
            default: break;
        }
        if (AB_BC(e_row >= 0 && e_row < sg.n_rows)) {
            if (sg.tag_out) st_tagged(sg.out, e_row, o, tag_of(epoch, sg.tag_out));
            else sg.out[e_row] = __float2half_rn(o);
        }
    }
}

}  // namespace ab
