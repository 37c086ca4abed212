"""From a model folder (or a configuration and a seed) to an :class:`Engine`."""

from __future__ import annotations

import os
from typing import Optional, Union

import torch

from ..cache.manager import PagedCache, bytes_per_token, plan_pool_tokens
from ..config.base import ModelConfig, architecture_of, load_config
from ..kernels import lib
from ..parts.base import Runtime
from ..weights.loader import load_weights, random_weights
from .model import DecoderModel
from .step import Engine

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
          "fp32": torch.float32}


def parse_dtype(d: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(d, torch.dtype):
        if d not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {d}")
        return d
    try:
        return DTYPES[d.lower()]
    except KeyError:
        raise ValueError(f"dtype '{d}' is not bfloat16 or float32") from None


def require_gpu(device: Union[str, torch.device]) -> torch.device:
    """The engine has no CPU path: the device must be a CUDA GPU and the kernels must load."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"axon_b200 runs on a CUDA GPU only (asked for '{device}')")
    if not torch.cuda.is_available():
        raise RuntimeError("axon_b200 needs a CUDA GPU and none is visible; there is no CPU fallback")
    lib.cuda()
    return dev


def step_workspace_bytes(hidden_size: int, vocab_size: int, max_step_tokens: int, max_slots: int) -> int:
    """An upper estimate of the scratch a step of ``max_step_tokens`` tokens takes beside weights
    and cache: the float32 residual, the normed copy, the mixer's and the feed-forward's
    intermediates (taken as 64 bytes per token and hidden element, about twice what the
    Qwen2 shapes use) and float32 logits for one wanted row per slot."""
    return max_step_tokens * hidden_size * 64 + 4 * vocab_size * max(max_slots, 1)


def build_engine(folder: Optional[str] = None, *, config: Optional[ModelConfig] = None,
                 seed: Optional[int] = None, dtype: Union[str, torch.dtype] = "bfloat16",
                 device: Union[str, torch.device] = "cuda:0", page_size: int = 16,
                 max_tokens: Optional[int] = 4096, max_slots: int = 16, max_positions: Optional[int] = None,
                 shuffle_seed: int = 0, max_step_tokens: int = 8192, gain_std: float = 0.1,
                 check_tables: Optional[bool] = None) -> Engine:
    """An engine over the model in ``folder`` (config.json + safetensors), or over seeded
    random weights of ``config`` made on the device when no folder is given.

    ``max_tokens`` sizes the cache pool (positions over all live requests, in whole
    pages); None takes what the device has free once the weights are placed, up to
    ``max_slots`` requests of ``max_positions`` (``plan_pool_tokens``).  ``max_slots`` is the
    number of live requests, ``max_positions`` the longest request (default: the model's
    ``max_position_embeddings``).  ``check_tables`` (default: the environment's
    ``AXON_CHECK_TABLES=1``) is a debugging mode in which the kernels compare every
    block-table entry they read with the pool's size and the step raises instead of
    following a bad one.
    """
    dev = require_gpu(device)
    dt = parse_dtype(dtype)
    if folder is not None:
        config = load_config(folder)
    elif config is None:
        raise ValueError("build_engine needs a model folder or a configuration")
    arch = architecture_of(config.to_dict())
    spec = arch.build_spec(config)
    rt = Runtime(dt, dev)
    with torch.cuda.device(dev):
        if folder is not None:
            weights = load_weights(folder, spec, dt, dev)
        else:
            weights = random_weights(spec, 0 if seed is None else seed, dt, dev, gain_std=gain_std)
        model = DecoderModel(spec, weights, rt)
        del weights
        max_positions = max_positions or spec.max_positions
        if max_tokens is None:
            torch.cuda.synchronize(dev)
            torch.cuda.empty_cache()            # what loading set free counts as free
            free, _ = torch.cuda.mem_get_info(dev)
            max_tokens = plan_pool_tokens(free, bytes_per_token(model.needs, dt), page_size, max_slots, max_positions,
                                          step_workspace_bytes(spec.hidden_size, spec.vocab_size,
                                                               min(max_step_tokens, max_slots * max_positions), max_slots))
            if max_tokens < page_size:
                raise RuntimeError(f"{free >> 20} MiB are free on {dev} once the weights are placed: no room for a cache pool")
        if check_tables is None:
            check_tables = os.environ.get("AXON_CHECK_TABLES", "0") not in ("", "0")
        cache = PagedCache(model.needs, dt, dev, page_size=page_size, max_tokens=max_tokens,
                           max_slots=max_slots, max_positions=max_positions,
                           shuffle_seed=shuffle_seed, check_tables=check_tables)
    engine = Engine(model, cache, max_step_tokens=max_step_tokens)
    engine.config = config
    return engine
