// Device-side storage of quantized matrices ("cell planes").
//
// The reference keeps weights in 16-row stripes tuned for NEON `tbl`/`sdot`
// (src/kernels/simd_lut.rs:3264-3400 for bit-planes, 4796-5023 for NF).  On the GPU the unit is the
// CELL: one row x one 64-column chunk, owned by one lane.  A warp takes 32 consecutive chunks of a
// row per step (lane l = chunk l), so cells are stored row-major, [row][chunk], and a warp step reads
// 32 x 32 B = 1 KiB of contiguous weights with 128-bit loads.  A lane keeps the int8 activations of
// its chunk in registers for all the rows it visits.
//
// The image is a sequence of up to three code planes and a scale plane.  Every plane is cut into PASS TILES: tile p
// holds chunks 32p .. 32p+n_p-1 (n_p = 32, fewer in the last tile) of ALL rows, [row][n_p cells], so the cells a warp
// needs for a 4-row block of one pass are one contiguous run of 4 x n_p x cell bytes - one bulk copy per plane, 2 KiB
// for a full pass of 16-byte cells.  (Row-major planes would give four 512-byte runs per plane for every matrix wider
// than 32 chunks, and the copy engine's rate of small copies, not HBM, then bounds the kernel.)  Rows are padded to a
// multiple of 4 with zero cells.  Tile p of a plane starts p x rows_pad x 32 x cell bytes into the plane.
//   bit-planes b4/b5/b6:  plane 0 / plane 1, 16 B/cell: low 4 bits of columns 0..31 / 32..63; word w
//                         (8 columns): byte b holds column 8w+b in its low nibble and column 8w+4+b in its
//                         high nibble (`word & 0x0F0F0F0F` = columns 8w..8w+3, `& 0xF0F0F0F0` = 8w+4.., x16)
//                         b5: plane 2, 8 B/cell: word h (columns 32h..): bit 8*(col%4) + (col%32)/4
//                         b6: plane 2, 16 B/cell: word v (columns 16v..): bits 8*(col%4) + 2*((col%16)/4), 2 wide
//   NF4 / NF5:            plane 0 / plane 1, 16 B/cell: word w = eight consecutive nibbles, nibble k = column
//                         8w+k (consecutive nibbles are `prmt` selectors); NF5 plane 2, 8 B/cell as for b5
//   NF3:                  plane 0, 16 B/cell (words W0..W3), plane 1, 8 B/cell (W4, W5): columns 0..47 sit
//                         in the low three bits of nibble col%8 of word col/8; column 48+t (t<16) has
//                         index bit j in bit 3 of nibble t%8 of word 3*(t/8)+j
//   E8Q2:                 plane 0, 16 B/cell: byte 2*blk = template byte, 2*blk+1 = sign byte of columns 8blk..
// Scales: bf16, in pass tiles as well: tile p holds, for every row, the scale groups that chunks 32p .. 32p+n_p-1
// touch (a group that straddles two passes is stored in both), row pitch = those groups x 2 bytes rounded up to 4;
// tile p starts p x rows_pad x 64 bytes into the scale plane.
// NF4 indices are re-encoded at upload: the 16 centroids are sorted ascending and the stored nibble is
// the rank of the centroid, so bit 3 of a nibble separates the eight largest from the eight smallest
// centroids (identity for the sorted codebooks the reference compiler emits).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/kronos_cuda_ffi.h"

namespace k2t {

enum Format : uint32_t { FMT_BP4 = 0, FMT_BP5, FMT_BP6, FMT_NF4, FMT_NF3, FMT_NF5, FMT_E8Q2, FMT_COUNT };

// ---- pass-tile addressing (host and device)
#ifdef __CUDACC__
#define K2T_HD __host__ __device__
#else
#define K2T_HD
#endif
K2T_HD inline uint32_t tile_chunks(uint32_t nc, uint32_t p) { return nc - 32u * p < 32u ? nc - 32u * p : 32u; }
K2T_HD inline size_t tile_code_off(uint32_t rows_pad, uint32_t cell, uint32_t p) { return (size_t)p * rows_pad * 32u * cell; }
K2T_HD inline uint32_t tile_scale_pitch(uint32_t nc, uint32_t sgc, uint32_t p) {     // bytes per row of scale tile p
    const uint32_t g_lo = (32u * p) / sgc, g_hi = (32u * p + tile_chunks(nc, p) - 1u) / sgc;
    return ((g_hi - g_lo + 1u) * 2u + 3u) & ~3u;
}
K2T_HD inline size_t tile_scale_off(uint32_t rows_pad, uint32_t p) { return (size_t)p * rows_pad * 64u; }

struct MatrixGeom {
    Format fmt;
    uint32_t rows, cols, nc, sgc, nsg;
    uint32_t rows_pad;        // rows rounded up to 4
    uint32_t np;              // pass tiles: ceil(nc / 32)
    uint32_t cell[3];         // bytes per cell of each code plane (0 = plane absent)
    int32_t max_odd;          // 2^B - 1 for bit-planes, 0 otherwise
    int8_t codebook32[32];    // expanded codebook (NF; NF4: sorted ascending), zero otherwise
    uint8_t nf4_rank[16];     // NF4: file index -> device nibble
    int32_t nf4_split_ok;     // NF4: 1 when the two-table decode applies (see k2t_gemv.cu)
    int32_t nf4_offset;       // NF4 two-table decode: centroid = table value + offset
    uint8_t nf4_hi[8];        // codebook32[8+l] - offset   (0..127)
    uint8_t nf4_lo[8];        // offset - codebook32[l]     (0..127)
    size_t plane_off[3];      // byte offsets of the code planes in the image
    size_t scale_off;         // byte offset of the scale plane
    size_t image_total;       // bytes of the whole image (16 bytes of slack after the last plane)
    size_t file_bytes;        // bytes of the matrix in the reference file format
    size_t image_bytes() const { return image_total; }
    // byte offsets of cell (row, chunk c) in plane k and of its scale in the image
    size_t cell_off(int k, uint32_t row, uint32_t c) const {
        const uint32_t p = c / 32;
        return plane_off[k] + tile_code_off(rows_pad, cell[k], p) + ((size_t)row * tile_chunks(nc, p) + c % 32) * cell[k];
    }
    size_t scale_off_of(uint32_t row, uint32_t c) const {
        const uint32_t p = c / 32;
        return scale_off + tile_scale_off(rows_pad, p) + (size_t)row * tile_scale_pitch(nc, sgc, p) + (size_t)(c / sgc - (32u * p) / sgc) * 2;
    }
};

// Validates `d` and fills `g`. Returns false and sets `err` on a malformed descriptor.
bool matrix_geometry(const KronosCudaMatrixDesc &d, MatrixGeom &g, std::string &err);

// Builds the device image (code planes, scales) in `out` (size g.image_bytes()).
void repack_matrix(const KronosCudaMatrixDesc &d, const MatrixGeom &g, bool gate_up_interleave,
                   uint8_t *out, unsigned threads);

}  // namespace k2t
