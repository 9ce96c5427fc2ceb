"""Shared helpers of the parity tests: torch <-> oracle array conversion and seeded inputs."""
import numpy as np
import torch

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
ID_NP = {"u8": np.uint8, "u32": np.uint32, "i64": np.int64}
ID_TORCH = {"u8": torch.uint8, "u32": torch.uint32, "i64": torch.int64}


def to_oracle(t: torch.Tensor) -> np.ndarray:
    """torch tensor (any device) -> the array layout the oracle takes (uint16 bits for f16/bf16)."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        return t.numpy()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def from_oracle(a: np.ndarray, dtype: str, device="cuda") -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if dtype == "f32":
        return torch.from_numpy(a).to(device)
    return torch.from_numpy(a.view(np.int16)).view(TORCH_DT[dtype]).to(device)


def ids_tensor(ids: np.ndarray, device="cuda") -> torch.Tensor:
    ids = np.ascontiguousarray(ids)
    if ids.dtype == np.uint32:
        return torch.from_numpy(ids.view(np.int32)).view(torch.uint32).to(device)
    return torch.from_numpy(ids).to(device)


def bits(t: torch.Tensor) -> np.ndarray:
    """Bit patterns for exact comparison."""
    a = to_oracle(t)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def randn(rng, shape, dtype: str, mean=0.0, std=1.0) -> np.ndarray:
    """Seeded N(mean, std) rounded to `dtype`, in oracle layout."""
    import oracle

    x = (mean + std * rng.standard_normal(shape)).astype(np.float32)
    return x if dtype == "f32" else oracle.cast_from_f32(x, dtype)


def make_qtable(rng, qtype: str, vocab: int, hidden: int) -> np.ndarray:
    """Raw block bytes [vocab, hidden/32*block_bytes] with the value distributions of the
    benchmark configs: f16 scale |N(0,0.01)|, int8 quants uniform[-127,127] (Q8_0) or 4-bit
    quants uniform[0,15]; the formats with a minimum get m ~ N(0,0.05) in f16, the 5-bit formats
    32 uniform high bits."""
    nb = hidden // 32
    d = np.abs(rng.standard_normal((vocab, nb)) * 0.01).astype(np.float16)
    parts = [d.view(np.uint8).reshape(vocab, nb, 2)]
    if qtype in ("q4_1", "q5_1"):
        m = (rng.standard_normal((vocab, nb)) * 0.05).astype(np.float16)
        parts.append(m.view(np.uint8).reshape(vocab, nb, 2))
    if qtype in ("q5_0", "q5_1"):
        parts.append(rng.integers(0, 256, size=(vocab, nb, 4), dtype=np.int16).astype(np.uint8))
    if qtype == "q8_0":
        parts.append(rng.integers(-127, 128, size=(vocab, nb, 32), dtype=np.int16).astype(np.int8).view(np.uint8))
    else:
        parts.append(rng.integers(0, 256, size=(vocab, nb, 16), dtype=np.int16).astype(np.uint8))
    blocks = np.concatenate(parts, axis=2)
    return np.ascontiguousarray(blocks.reshape(vocab, -1))


def _oracle():
    import oracle

    return oracle


def make_kq_blocks(rng, qtype, n_blocks):
    """Random but well-formed super-blocks: every byte uniform, the f16 / f32 scales |N(0, 0.01)|."""
    bb = _oracle().BLOCK_BYTES[qtype]
    raw = rng.integers(0, 256, size=(n_blocks, bb), dtype=np.int16).astype(np.uint8)
    d = np.abs(rng.standard_normal((n_blocks, 2)) * 0.01).astype(np.float16).view(np.uint8).reshape(n_blocks, 4)
    if qtype == "q2k":
        raw[:, 80:84] = d
    elif qtype == "q3k":
        raw[:, 108:110] = d[:, :2]
    elif qtype in ("q4k", "q5k"):
        raw[:, 0:4] = d
    elif qtype == "q6k":
        raw[:, 208:210] = d[:, :2]
    else:
        raw[:, 0:4] = np.abs(rng.standard_normal(n_blocks) * 0.01).astype(np.float32).view(np.uint8).reshape(n_blocks, 4)
    return raw


def stable_seed(*parts) -> int:
    """A seed that depends only on the test's parameters (Python's own hash() of a string changes from
    one process to the next)."""
    import zlib

    return zlib.crc32(repr(parts).encode())
