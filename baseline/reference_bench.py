"""`bench.py --impl reference`.

The reference cannot be installed as a package in this environment:
``pip install --no-index --no-build-isolation --find-links /opt/wheelhouse --target baseline/_ref
<reference>`` stops while generating metadata (its setup.py imports ``setuptools_scm``, which is
neither installed nor in the wheelhouse), and past that point its extension links the closed
``libaccl_barex.so`` (+ libibverbs) that the image does not have, while its Python control plane
imports a vLLM fork.  So the public API of the reference is unavailable and this arm says so.

What can be measured is the reference's own intra-box data path, compiled UNMODIFIED from its
sources into ``baseline/_ref/ref_datapath``: its ParseBlock generator and its copy kernels,
gather GPU -> pinned host then scatter pinned host -> GPU, with the socket hop of its TCP channel
left out.  That number is attached as ``partial`` (an upper bound on the reference), next to the
``unavailable`` line the contract asks for.  The reference has no cross-layout transfer, so the
partial number is NHD -> NHD.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
BIN = os.path.join(REF_DIR, "ref_datapath")
WHY = ("reference not installable offline: setup.py needs setuptools_scm (absent from the wheelhouse) and its "
       "extension links the closed libaccl_barex.so + libibverbs; the control plane needs a vLLM fork")


def reference_checkout() -> str:
    """Where the reference's sources are: LLUMNIX_KV_REFERENCE, else a ``reference`` folder next to this
    repository's checkout."""
    env = os.environ.get("LLUMNIX_KV_REFERENCE")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference_root: str = "", verbose: bool = False) -> str:
    """Compile the reference's own sources (unmodified, read in place) plus the harness."""
    reference_root = reference_root or reference_checkout()
    root = os.path.join(reference_root, "kvtransfer")
    if not os.path.isdir(root):
        raise RuntimeError("no reference checkout to build the data path from")
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    inc = [f"-I{root}/include", f"-I{root}/src", "-I/usr/local/cuda/include"]
    objs = []
    # the reference's CMake builds compute_100 (generic), not sm_100a: keep that
    cu = os.path.join(REF_DIR, "copy_kernels.cu.o")
    cmds = [[nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100,code=sm_100", *inc, "-c",
             f"{root}/src/copy_kernels.cu", "-o", cu]]
    objs.append(cu)
    for src in ("copy_kernels", "envcfg", "third_party/logging", "parse_block_common", "parse_block_flash", "common"):
        o = os.path.join(REF_DIR, src.replace("/", "_") + ".o")
        cmds.append(["g++", "-std=c++17", "-O2", "-DNDEBUG", *inc, "-c", f"{root}/src/{src}.cpp", "-o", o])
        objs.append(o)
    main_o = os.path.join(REF_DIR, "main.o")
    cmds.append(["g++", "-std=c++17", "-O2", "-DNDEBUG", *inc, "-c", os.path.join(HERE, "ref_datapath_main.cpp"),
                 "-o", main_o])
    objs.append(main_o)
    cmds.append([nvcc, "-o", BIN, *objs, "-lpthread", "-lrt"])
    for c in cmds:
        r = subprocess.run(c, capture_output=True, text=True)
        if verbose:
            print(" ".join(c), r.stdout, r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"reference data path did not build: {' '.join(c)}\n{r.stderr[-800:]}")
    return BIN


def main(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    out = {"impl": "reference", "unavailable": WHY}
    partial = None
    try:
        if not os.path.isfile(BIN):
            build()
        n_pairs = max(1, world // 2)
        ms, nbytes, ok = 0.0, 0, True
        if rank < n_pairs:
            src = rank
            dst = rank + n_pairs if world > 1 else rank
            layers = 4 if args.small else args.layers
            tokens = 2048 if args.small else args.tokens
            r = subprocess.run([BIN, str(src), str(dst), str(layers), str(tokens), str(args.requests), str(args.slots),
                                str(args.warmup), str(args.steps)], capture_output=True, text=True, timeout=1200)
            if r.returncode != 0:
                raise RuntimeError(f"ref_datapath exit {r.returncode}: {r.stderr[-300:]}")
            f = r.stdout.strip().splitlines()[-1].split()   # the reference prints its env settings first
            ms, nbytes, ok = float(f[0]), int(f[1]), f[2] == "1"
        if world > 1:
            import torch
            import torch.distributed as dist

            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dist.init_process_group("nccl")
            t = torch.tensor([ms, float(nbytes), float(ok)], dtype=torch.float64, device="cuda")
            mx = t.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            mn = t.clone()
            dist.all_reduce(mn, op=dist.ReduceOp.MIN)
            ms, nbytes = float(mx[0]), int(mx[1])
            okv = torch.tensor([1.0 if (ok or rank >= n_pairs) else 0.0], device="cuda")
            dist.all_reduce(okv, op=dist.ReduceOp.MIN)
            ok = bool(okv.item())
            dist.destroy_process_group()
        gbps = n_pairs * nbytes * args.steps / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
        partial = {"what": "reference ParseBlock + copy kernels, gather D2H -> pinned host -> scatter H2D, no socket hop; "
                           "NHD->NHD (the reference has no cross-layout path); upper bound on the reference intra-box",
                   "metric": "p2d_kv_transfer_GBps", "value": round(gbps, 2), "unit": "GB/s", "n_gpus": world,
                   "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / max(1, args.steps), 4),
                   "verified": ok}
    except Exception as ex:   # the arm must always answer
        partial = {"error": f"{type(ex).__name__}: {ex}"[:300]}
    out["partial"] = partial
    if rank == 0:
        print(json.dumps(out))


if __name__ == "__main__":
    build(verbose="-v" in sys.argv)
    print(BIN)
