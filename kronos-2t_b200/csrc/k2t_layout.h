// Device-side storage of quantized matrices ("cell planes").
//
// The reference keeps weights in 16-row stripes tuned for NEON `tbl`/`sdot`
// (src/kernels/simd_lut.rs:3264-3400 for bit-planes, 4796-5023 for NF).  On the GPU the unit is the
// CELL: one row x one 64-column chunk, owned by one lane.  A warp takes 32 consecutive chunks of a
// row per step (lane l = chunk l), so cells are stored row-major, [row][chunk], and a warp step reads
// 32 x 32 B = 1 KiB of contiguous weights with 128-bit loads.  A lane keeps the int8 activations of
// its chunk in registers for all the rows it visits.
//
// The image is a sequence of up to three code planes and a scale plane.  A plane is [rows] x [row
// pitch] bytes; the pitch is the cells of a row (nc x cell bytes) rounded up to 16 so that every row
// and every 32-chunk pass of a row starts on a 16-byte boundary (bulk-copy granularity):
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
// Scales: bf16 [rows][nsg_pad], nsg_pad = scale groups per row rounded up to 8 (16-byte rows).
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

struct MatrixGeom {
    Format fmt;
    uint32_t rows, cols, nc, sgc, nsg, nsg_pad;
    uint32_t cell[3];         // bytes per cell of each code plane (0 = plane absent)
    uint32_t pitch[3];        // bytes per row of each code plane (multiple of 16)
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
};

// Validates `d` and fills `g`. Returns false and sets `err` on a malformed descriptor.
bool matrix_geometry(const KronosCudaMatrixDesc &d, MatrixGeom &g, std::string &err);

// Builds the device image (code planes, scales) in `out` (size g.image_bytes()).
void repack_matrix(const KronosCudaMatrixDesc &d, const MatrixGeom &g, bool gate_up_interleave,
                   uint8_t *out, unsigned threads);

}  // namespace k2t
