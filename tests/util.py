"""Helpers shared by the test modules."""
import numpy as np
import torch

from oracle import nvfp4_oracle as O


def bf16_np_to_torch(bits: np.ndarray, device="cuda") -> torch.Tensor:
    """uint16 bf16 bit patterns -> torch.bfloat16 tensor."""
    return torch.from_numpy(bits.astype(np.int16, copy=True).reshape(bits.shape)).view(torch.bfloat16).to(device)


def f32_np_to_bf16_torch(x: np.ndarray, device="cuda") -> torch.Tensor:
    return bf16_np_to_torch(O.bf16_bits(x), device)


def torch_bf16_to_f32_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def torch_bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().cpu().view(torch.uint8).numpy()


def config_activation(m: int, k: int, seed: int = 0) -> torch.Tensor:
    """~N(0,1) with 0.1 % of entries scaled x20 (the benchmark's activation distribution), bf16, CPU."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    mask = torch.rand(m, k, generator=g) < 0.001
    return torch.where(mask, x * 20, x).bfloat16()


def config_weight(n: int, k: int, seed: int = 1) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, k, generator=g) * 0.02).bfloat16()
