#!/usr/bin/env python3
"""Node preflight: what the research harness needs from a machine, checked in one command.

The original project ships cloud provisioning (GCP instances, a Slurm image with CUDA, NCCL,
OpenMPI and a bit-packing extension, and an MPI all-reduce smoke test:
paper-code/environment/cluster.py, files/setup.sh, mpi_test.py). A B200 node needs none of that
software stack built; what remains useful is the smoke test and a report of what the node
offers. Launch it like a training job:

    python -m torch.distributed.run --nproc-per-node 8 -m powersgd_b200.paper.environment
    python -m powersgd_b200.paper.environment            # single process: report only

Every rank checks (read-only; no GPU setting is changed): the native library and its exported
entry points, CUDA device / compute capability, peer access to every other local GPU, a
library all-reduce, and (CUDA, world > 1) this library's in-kernel all-reduce over peer memory.
Rank 0 prints one JSON report; the exit code is non-zero when a required check failed.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist


def _native_report() -> dict:
    try:
        from ..ops import native

        lib = native.lib()
        return {"ok": True, "path": getattr(lib, "_name", "?"), "max_rank": int(lib.psgd_gemm_template_rank(1 << 10))}
    except Exception as exc:  # not built, or not loadable on this machine
        return {"ok": False, "error": str(exc)[:200]}


def _device_report(local: int) -> dict:
    if not torch.cuda.is_available():
        return {"cuda": False}
    props = torch.cuda.get_device_properties(local)
    peers = [bool(torch.cuda.can_device_access_peer(local, j)) for j in range(torch.cuda.device_count()) if j != local]
    return {
        "cuda": True, "name": props.name, "capability": f"{props.major}.{props.minor}", "sms": props.multi_processor_count,
        "memory_gib": round(props.total_memory / 2**30, 1), "local_gpus": torch.cuda.device_count(),
        "peer_access_to_all": all(peers) if peers else True,
    }


def main(backend: str | None = None) -> dict:
    distributed = "RANK" in os.environ
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if cuda else "gloo")
    device = torch.device("cuda", local) if (cuda and backend == "nccl") else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(local)
    report = {"world": world, "backend": backend, "torch": torch.__version__, "native": _native_report(),
              "device": _device_report(local), "checks": {}}
    ok = True
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if not dist.is_initialized():
            kwargs = {"device_id": device} if device.type == "cuda" else {}
            dist.init_process_group(backend, **kwargs)
        # the smoke test of the original (an all-reduce of ones must give the world size everywhere)
        x = torch.ones(1 << 16, device=device)
        dist.all_reduce(x)
        good = bool((x == world).all())
        report["checks"]["library_all_reduce"] = good
        ok = ok and good
        if device.type == "cuda" and world > 1 and report["native"]["ok"]:
            from ..parallel.symm import Channel

            ch = Channel(1 << 16, timeout_ms=5000)
            y = torch.full((1 << 16,), float(rank + 1), device=device)
            ch.all_reduce_(y)
            torch.cuda.synchronize()
            good = ch.status == 0 and bool((y == world * (world + 1) / 2).all())
            report["checks"]["in_kernel_all_reduce"] = good
            ok = ok and good
            ch.close()
        flags = torch.tensor([1.0 if ok else 0.0], device=device)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        ok = bool(flags.item() == 1.0)
    if device.type == "cuda":
        ok = ok and report["native"]["ok"]  # on a GPU node the kernels are the product
    report["ok"] = ok
    if rank == 0:
        print(json.dumps(report))
    return report


if __name__ == "__main__":
    result = main()
    if dist.is_initialized():
        dist.destroy_process_group()
    sys.exit(0 if result["ok"] else 1)
