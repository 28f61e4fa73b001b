"""Synthetic matrices in the reference's file formats, built without any quantizer: uniformly random
codes / indices and bf16 scales in [2^-15, 2^-7).  GEMV time does not depend on the code values;
files produced this way are valid inputs for kronos_cuda_matrix_upload (and for the oracle)."""
import numpy as np

NF4_DEFAULT = np.array([-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127], np.int8)
NF3_DEFAULT = np.array([-127, -79, -45, -14, 14, 45, 79, 127, 0, 0, 0, 0, 0, 0, 0, 0], np.int8)
_NF_CHUNK = {5: 640, 4: 512, 3: 384, 2: 256}


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def random_bipolar_bytes(seed, rows, cols, planes):
    """(interleaved planes u8, bf16 scales u16) of a FusedBipolarLutMatrix with random codes."""
    ns, nc = (rows + 15) // 16, cols // 64
    rng = _rng(seed)
    data = rng.integers(0, 256, ns * (cols // 8) * planes * 16, dtype=np.uint8)
    scales = rng.integers(0x3800, 0x3C00, ns * nc * 16, dtype=np.uint16)
    return data, scales


def random_nf_bytes(seed, rows, cols, bits, sgc):
    """(pair_stream, tail_stream) of an NfSdotMatrix with random indices; rows % 32 == 0, (cols/64) % sgc == 0."""
    nc = cols // 64
    assert rows % 32 == 0 and nc % sgc == 0
    nsg, cb = nc // sgc, _NF_CHUNK[bits]
    rng = _rng(seed)
    blk = 64 + sgc * 2 * cb
    stream = rng.integers(0, 256, (rows // 32) * nsg * blk, dtype=np.uint8).reshape(rows // 32, nsg, blk)
    sc = rng.integers(0x3800, 0x3C00, (rows // 32, nsg, 32), dtype=np.uint16)
    stream[:, :, :64] = sc.view(np.uint8).reshape(rows // 32, nsg, 64)
    return stream.reshape(-1), np.zeros(0, np.uint8)


def file_bytes(kind, rows, cols, bits, sgc=1):
    """Bytes of a matrix in the reference file format (the algorithmic weight bytes of one GEMV)."""
    ns, nc = (rows + 15) // 16, cols // 64
    if kind == "bipolar":
        return ns * (cols // 8) * bits * 16 + ns * nc * 16 * 2
    nsg, cb = -(-nc // sgc), _NF_CHUNK[bits]
    return (ns // 2) * (nsg * 64 + nc * 2 * cb) + (ns & 1) * (nsg * 32 + nc * cb) + 16
