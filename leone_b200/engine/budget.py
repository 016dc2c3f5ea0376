"""The memory budget: what an engine will hold on the device, checked before anything is uploaded.

The reference sums the model's tensor bytes and refuses to load when they exceed what the
backend reports as available (``check_weight_budget`` → ``WeightBudget{required_bytes,
available_bytes}``, crates/leone/src/model.rs:350-366).  Here the sum also holds what the
engine allocates right after the weights, because its sizes are known from the arguments:
the page pools, the fixed-size state of every slot, the most one part holds on top of its
tensors while it loads (a fused copy beside its sources) and the scratch buffers that are
sized by ``max_batch_tokens``.  The last item is an estimate; the others are exact.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import torch

from ..weights.loader import target_dtype


class WeightBudgetError(MemoryError):
    """The model, its cache and its scratch do not fit into the device's free memory."""

    def __init__(self, required_bytes: int, available_bytes: int, plan: Dict[str, int]):
        self.required_bytes = int(required_bytes)
        self.available_bytes = int(available_bytes)
        self.plan = dict(plan)
        gib = 2.0 ** 30
        parts = ", ".join(f"{k} {v / gib:.2f}" for k, v in plan.items() if k != "required")
        super().__init__(
            f"memory budget: the engine needs {required_bytes} bytes ({required_bytes / gib:.2f} GiB: {parts}) "
            f"but the device has {available_bytes} bytes ({available_bytes / gib:.2f} GiB) available; "
            "nothing was loaded")


def _itemsize(dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def plan_memory(model, specs, stored_dtypes: Optional[Dict[str, torch.dtype]], run_dtype, group_specs,
                num_pages: int, page_tokens: int, state_shapes: Dict[int, Sequence[int]], max_requests: int,
                max_batch_tokens: int) -> Dict[str, int]:
    """Bytes by class: ``weights`` (every tensor in the dtype it will be kept in), ``load``
    (transient), ``cache`` (page pools of all groups), ``state`` (fixed-size slots),
    ``scratch`` (estimate), and their sum ``required``."""
    weights = 0
    for spec in specs:
        stored = (stored_dtypes or {}).get(spec.name, torch.float32)
        numel = 1
        for d in spec.shape:
            numel *= int(d)
        weights += numel * _itemsize(target_dtype(spec, stored, run_dtype))
    cache = 0
    for gs in group_specs:
        k_el, v_el = gs.page_elements(page_tokens)
        cache += len(gs.layers) * num_pages * (k_el + v_el) * _itemsize(gs.dtype or run_dtype)
    state = 0
    for shape in state_shapes.values():
        n = 4
        for d in shape:
            n *= int(d)
        state += n
    plan = dict(weights=weights, load=model.load_transient_bytes(), cache=cache, state=state,
                scratch=model.scratch_bytes(max_batch_tokens, 2 * max_requests))
    plan["required"] = sum(plan.values())
    return plan


def device_free_bytes(device) -> Optional[int]:
    """Free bytes of a CUDA device as an allocation through torch sees them: what the driver
    reports free plus what torch's caching allocator holds without using it.  ``None`` where
    there is no such figure (a CPU device)."""
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        return None
    free, _total = torch.cuda.mem_get_info(device)
    cached = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    return int(free + max(cached, 0))


def check_memory_budget(plan: Dict[str, int], device, free_bytes: Optional[Callable[[], int]] = None) -> None:
    """Raise :class:`WeightBudgetError` if ``plan['required']`` exceeds the free bytes."""
    available = free_bytes() if free_bytes is not None else device_free_bytes(device)
    if available is None:
        return
    if plan["required"] > available:
        raise WeightBudgetError(plan["required"], available, plan)
