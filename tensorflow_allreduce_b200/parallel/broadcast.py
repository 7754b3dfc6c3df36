"""Make every rank start from (or resume with) the same weights and optimizer state.

The reference has no broadcast: its ranks must build identical variables from a fixed seed
(`tensorflow/contrib/mpi_collectives/mpi_ops_test.py:92`) or all restore the same checkpoint
file. These helpers let one rank load a plain `state_dict` and hand it to the others. The
library keeps no checkpoint format of its own.
"""
from __future__ import annotations

from typing import Dict, Iterable, Union

import torch

from .. import core


def _named_tensors(obj) -> Dict[str, torch.Tensor]:
    if isinstance(obj, torch.nn.Module):
        return dict(obj.state_dict(keep_vars=True))
    if isinstance(obj, dict):
        return {k: v for k, v in obj.items() if isinstance(v, torch.Tensor)}
    return {str(i): t for i, t in enumerate(obj)}


@torch.no_grad()
def broadcast_parameters(params: Union[torch.nn.Module, Dict[str, torch.Tensor], Iterable[torch.Tensor]], root: int = 0,
                         name: str = "broadcast_parameters") -> None:
    """Overwrite every tensor (parameters and buffers of a module, or the tensors of a dict / list)
    with its value on rank `root`. Tensors are packed per (device, dtype) so that a model costs a
    handful of collectives, not one per tensor. Every rank must pass the same structure."""
    named = _named_tensors(params)
    groups: Dict[tuple, list] = {}
    for k in sorted(named):
        t = named[k]
        if t.numel() == 0:
            continue
        groups.setdefault((str(t.device.type), str(t.dtype)), []).append(t)
    for gi, key in enumerate(sorted(groups)):
        ts = groups[key]
        dtype = ts[0].dtype
        wire = dtype if dtype in core._DTYPES else None
        flat = torch.cat([t.detach().reshape(-1) for t in ts])
        if wire is None:
            flat = flat.view(torch.uint8) if dtype != torch.bool else flat.to(torch.uint8)
        out = core.broadcast(flat, root=root, name=f"{name}.{gi}")
        if wire is None:
            out = out.view(dtype) if dtype != torch.bool else out.to(torch.bool)
        pos = 0
        for t in ts:
            n = t.numel()
            t.copy_(out[pos:pos + n].view(t.shape))
            pos += n


@torch.no_grad()
def broadcast_optimizer_state(optimizer: torch.optim.Optimizer, root: int = 0, name: str = "broadcast_optimizer_state") -> None:
    """Give every rank the optimizer state (`state_dict()`) of rank `root`. Tensors travel through
    the collectives, everything else (step counts, hyper-parameters) through the control plane."""
    sd = optimizer.state_dict()
    # Non-tensor part first: it also tells the other ranks which tensors to expect.
    meta = None
    if core.rank() == root:
        meta = {
            "param_groups": sd["param_groups"],
            "state": {k: {kk: (("__tensor__", tuple(vv.shape), str(vv.dtype)) if isinstance(vv, torch.Tensor) else vv)
                          for kk, vv in v.items()} for k, v in sd["state"].items()},
        }
    meta = core.host_allgather(meta, name=name + ".meta")[root]
    device = None
    for g in optimizer.param_groups:
        for p in g["params"]:
            device = p.device
            break
        if device is not None:
            break
    tensors, new_state = {}, {}
    for k, v in meta["state"].items():
        new_state[k] = {}
        for kk, vv in v.items():
            if isinstance(vv, tuple) and len(vv) == 3 and vv[0] == "__tensor__":
                dtype = getattr(torch, vv[2].split(".")[-1])
                if core.rank() == root:
                    t = sd["state"][k][kk].detach().clone()
                else:
                    t = torch.zeros(vv[1], dtype=dtype, device=device if len(vv[1]) else "cpu")
                if t.dim() == 0:
                    # scalars (e.g. Adam's step) ride along in the metadata exchange
                    val = core.host_allgather(t.item() if core.rank() == root else None, name=f"{name}.s.{k}.{kk}")[root]
                    t = torch.tensor(val, dtype=dtype, device=t.device)
                else:
                    tensors[f"{k}.{kk}"] = t
                new_state[k][kk] = t
            else:
                new_state[k][kk] = vv
    if tensors:
        broadcast_parameters(tensors, root=root, name=name + ".t")
    optimizer.load_state_dict({"state": new_state, "param_groups": meta["param_groups"]})
