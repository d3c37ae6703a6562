// Push schedule of the all-gather GEMM's comm CTAs: which bytes of this rank's quantized rows go where, in which
// order, and which arrival flag each unit raises.  Plain integer arithmetic shared by the kernel (gemm.cu) and by a
// host-side enumeration (tkb_debug_ag_schedule) that the CPU tests use to check coverage.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define TKB_HD __host__ __device__ __forceinline__
#else
#define TKB_HD inline
#endif

namespace tkb {

constexpr int kAgPartsPerBlock = 4;          // comm CTAs / copy engines: a 256-row block travels as 4 independently flagged 64-row parts
constexpr int kAgPartsPushWarps = 16;        // push warps in every CTA of the GEMM: 16-row parts, so that even 8 ranks' worth of units
                                             // ((world - 1) * M / world / 16) is a few per CTA
constexpr int kAgMaxParts = 32;              // the arrival arrays hold this many flags per 256 gathered rows
constexpr int kAgFanOut = 4;                 // destinations served at the same time.  SM-issued stores to ONE peer stop at about
                                             // 220-250 GB/s however many SMs issue them (measured with 20 comm CTAs and with the push
                                             // warps of all 148), so one destination at a time cannot fill the links; four can
constexpr int kAgFanOutPushWarps = 4;        // measured at 8 GPUs, M=8192 N=28672 K=8192: 195 us per step with 4, 234 us with 1

struct AgGeometry { int rank, world, blocks_per_rank, k_bytes, sc_bytes_per_mblock, parts, fan; };      // parts: flagged parts per 256-row block (4 or 16); fan: destinations served together
struct AgCursor { int u; int span; uint32_t o; };                 // unit, span (0 = codes, 1 = scales), bytes done in the span
struct AgPiece { size_t off; uint32_t bytes, span_len; int span, dst_rank, flag; };

// A unit is one part (256 / parts rows) of one of this rank's 256-row blocks for one destination.  Destinations are taken in the
// order in which they consume this rank's rows (rank-1 first), `fan` of them at a time; inside such a group the
// units alternate between the destinations, so consecutive comm CTAs write to different peers.
TKB_HD int ag_units(const AgGeometry& g) { return (g.world - 1) * g.blocks_per_rank * g.parts; }

// The next piece (at most piece_bytes) at the cursor.  `off` is a byte offset into the gathered codes (span 0) or
// scales (span 1) buffer, the same on the source and on the destination; `flag` indexes the arrival array.
TKB_HD AgPiece ag_piece(const AgGeometry& g, const AgCursor& c, uint32_t piece_bytes) {
    AgPiece pc;
    const int per_dst = g.blocks_per_rank * g.parts;
    const int part_rows = 256 / g.parts;
    const int first = (c.u / (g.fan * per_dst)) * g.fan;                  // first destination (consumption order) of the unit's group
    const int gsize = g.world - 1 - first < g.fan ? g.world - 1 - first : g.fan;
    const int v = c.u - first * per_dst;                                  // unit inside the group
    pc.dst_rank = (g.rank + g.world - 1 - (first + v % gsize)) % g.world;
    const int in_dst = v / gsize, b = in_dst / g.parts, part = in_dst % g.parts;
    const size_t row0 = (size_t(g.rank) * g.blocks_per_rank + b) * 256;
    pc.span = c.span;
    if (c.span == 0) {                       // codes of the part's rows: contiguous
        pc.span_len = uint32_t(part_rows) * uint32_t(g.k_bytes);
        pc.off = (row0 + size_t(part) * part_rows) * size_t(g.k_bytes) + c.o;
    } else {                                 // the part's share of the bytes of the block's two 128-row scale blocks (any split will
                                             // do: the consumer waits for every part of a block before it reads the block)
        pc.span_len = uint32_t(g.sc_bytes_per_mblock) * 2u / uint32_t(g.parts);
        pc.off = (row0 / 128) * size_t(g.sc_bytes_per_mblock) + size_t(part) * pc.span_len + c.o;
    }
    pc.bytes = piece_bytes < pc.span_len - c.o ? piece_bytes : pc.span_len - c.o;
    pc.flag = (g.rank * g.blocks_per_rank + b) * g.parts + part;
    return pc;
}

// Moves the cursor past a piece; true when that piece was the last of its unit (comm CTA i owns units i, i + n, ...).
TKB_HD bool ag_advance(AgCursor& c, const AgPiece& pc, int comm_ctas) {
    c.o += pc.bytes;
    if (c.o < pc.span_len) return false;
    c.o = 0;
    if (++c.span < 2) return false;
    c.span = 0;
    c.u += comm_ctas;
    return true;
}

} // namespace tkb
