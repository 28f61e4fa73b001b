"""Input generators of the reference's own kernel tests, restated (src/kernels/simd_lut.rs:9137-9175,
test_nf3_nf4_sdot_neon_scalar_parity_and_quality): a 64-bit LCG whose top 24 bits give uniform values in [-0.5, 0.5)."""
import numpy as np

M64 = (1 << 64) - 1


def sample_x(seed, cols):
    """Activation of the reference test: LCG(6364136223846793005, 1442695040888963407), every 23rd column six times larger."""
    s = (seed ^ 0x9E3779B97F4A7C15) & M64
    out = np.zeros(cols, np.float32)
    for c in range(cols):
        s = (s * 6364136223846793005 + 1442695040888963407) & M64
        u = np.float32(s >> 40) / np.float32(1 << 24) - np.float32(0.5)
        out[c] = u * np.float32(6.0 if c % 23 == 0 else 1.0)
    return out


def sample_weights(rows, cols):
    """Weights of the reference test: sum of two uniforms (heavy-ish tails) times 0.4, column 7 of every 64 scaled by 3.5."""
    ws = 0x517CC1B727220A95
    out = np.zeros(rows * cols, np.float32)
    for idx in range(rows * cols):
        ws = (ws * 6364136223846793005 + 1) & M64
        z1 = np.float32(ws >> 40) / np.float32(1 << 24) - np.float32(0.5)
        ws = (ws * 6364136223846793005 + 1) & M64
        z2 = np.float32(ws >> 40) / np.float32(1 << 24) - np.float32(0.5)
        out[idx] = (z1 + z2) * np.float32(0.4) * np.float32(3.5 if idx % 64 == 7 else 1.0)
    return out.reshape(rows, cols)
