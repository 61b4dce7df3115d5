"""The random-weights mode: writes a model folder (config.json and
model.safetensors) from a configuration and a seed.

Tensors are drawn in the order of their sorted names from one seeded CPU
generator, so a (configuration, seed, dtype) names one model.  Matrices and
tables are N(0, init_std), norm gains 1 + N(0, gain_std).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def random_tensors(expected, seed: int, dtype, init_std: float = 0.02, gain_std: float = 0.02,
                   device="cpu") -> dict[str, torch.Tensor]:
    dtype = _DTYPES[dtype]
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        if torch.device(device).type == "cuda":
            # a per-tensor seed drawn from the CPU generator keeps the order of names decisive
            s = int(torch.randint(0, 2 ** 62, (1,), generator=gen).item())
            g = torch.Generator(device=device).manual_seed(s)
            t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
        else:
            t = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        t = 1.0 + gain_std * t if spec.role == "gain" else init_std * t
        out[name] = t.to(dtype).contiguous()
    return out


def write_random_model(folder, config: Mapping[str, Any], seed: int = 0, dtype="bfloat16",
                       init_std: float = 0.02, gain_std: float = 0.02, device="cpu") -> Path:
    """Write ``folder/config.json`` and ``folder/model.safetensors``; return the folder."""
    from safetensors.torch import save_file

    from ..config import config_from_dict
    from ..engine.model import expected_weights

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(config)
    raw = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(config)
    raw["torch_dtype"] = "bfloat16" if _DTYPES[dtype] == torch.bfloat16 else "float32"
    (folder / "config.json").write_text(json.dumps(raw, indent=1) + "\n")
    tensors = random_tensors(expected_weights(cfg.model_spec()), seed, dtype, init_std, gain_std, device)
    save_file({k: v.cpu() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
