"""Process bootstrap for torchrun, mpiexec/mpirun and srun launches on NVIDIA nodes.

Same function names, arguments and result dictionaries as the reference's
sp_aurora/mpi_utils.py (detect_mpi_environment :16, get_mpi_info :35,
setup_distributed_environment :92, init_distributed_backend :164, cleanup_distributed :243,
get_device_for_rank :253, setup_mpi_distributed :293), built for one process per GPU:

* the launcher's variables are read from one table (Open MPI, PMI / Intel MPI / MPICH, PMIx,
  MVAPICH2, generic MPI_*, and Slurm's srun) and turned into RANK / WORLD_SIZE / LOCAL_RANK;
* the rendezvous address: MASTER_ADDR when given, the loopback address when every rank is on
  this node, the first host of the Slurm node list otherwise; a multi-node MPI launch without
  either is an error (the reference silently points non-zero ranks at localhost, :131-134);
* the backend defaults to NCCL on GPUs, bound to the rank's device (`device_id`, so the
  communicator is created eagerly) with high-priority streams, because the attention grids
  occupy every SM and a default-priority transfer kernel would wait for them; there is no
  silent fall-back from NCCL to gloo (the reference has one, :222-238): the ring and all-to-all
  paths need a GPU-capable backend, so a failed NCCL initialisation returns False;
* nothing is printed unless SPA_VERBOSE=1.
"""
from __future__ import annotations

import datetime
import os
import re
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

# launcher family -> (rank, world size, local rank, local size) variable names
_MPI_TABLE = (
    ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK",
     "OMPI_COMM_WORLD_LOCAL_SIZE"),
    ("PMI_RANK", "PMI_SIZE", "MPI_LOCALRANKID", "MPI_LOCALNRANKS"),
    ("PMIX_RANK", "PMIX_SIZE", "PMIX_LOCAL_RANK", "PMIX_LOCAL_SIZE"),
    ("MV2_COMM_WORLD_RANK", "MV2_COMM_WORLD_SIZE", "MV2_COMM_WORLD_LOCAL_RANK",
     "MV2_COMM_WORLD_LOCAL_SIZE"),
    ("MPI_RANK", "MPI_SIZE", "MPI_LOCAL_RANK", "MPI_LOCAL_SIZE"),
    ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID", "SLURM_NTASKS_PER_NODE"),
)
DEFAULT_PORT = 29500
LOOPBACK = "127.0.0.1"


def _say(msg: str) -> None:
    if os.environ.get("SPA_VERBOSE") == "1":
        print(f"[sp_aurora_b200] {msg}", flush=True)


def detect_mpi_environment() -> bool:
    """True when an MPI launcher's (or srun's) rank variable is present."""
    return any(row[0] in os.environ for row in _MPI_TABLE)


def _first_int(text: str, default: int) -> int:
    m = re.match(r"\s*(\d+)", text or "")
    return int(m.group(1)) if m else default


def get_mpi_info() -> Dict[str, Any]:
    """rank / world_size / local_rank / local_size from the launcher's variables (None when no
    launcher is detected). A missing local rank is 0 and a missing local size 1, as in the
    reference (:51-83)."""
    env = os.environ
    for rank_v, size_v, lrank_v, lsize_v in _MPI_TABLE:
        if rank_v not in env:
            continue
        size = env.get(size_v)
        if size is None and rank_v == "MPI_RANK":
            size = env.get("MPI_WORLD_SIZE", "1")
        return {"rank": int(env[rank_v]),
                "world_size": int(size) if size is not None else None,
                "local_rank": int(env.get(lrank_v, "0")),
                # Slurm writes forms like "8(x2)"
                "local_size": _first_int(env.get(lsize_v, "1"), 1)}
    return {"rank": None, "world_size": None, "local_rank": None, "local_size": None}


def first_slurm_host(nodelist: str) -> Optional[str]:
    """First host name of a Slurm node list ("node[03-05,9],x1" -> "node03")."""
    if not nodelist:
        return None
    m = re.match(r"([^,\[]+)(?:\[([^\]]+)\])?", nodelist.strip())
    if not m:
        return None
    prefix, ranges = m.group(1), m.group(2)
    if not ranges:
        return prefix
    return prefix + re.split(r"[,-]", ranges)[0]


def _master_addr(info: Dict[str, Any]) -> str:
    addr = os.environ.get("MASTER_ADDR")
    if addr:
        return addr
    if info["world_size"] is not None and info["local_size"] >= info["world_size"]:
        return LOOPBACK                                   # every rank lives on this node
    host = os.environ.get("SLURM_LAUNCH_NODE_IPADDR") or \
        first_slurm_host(os.environ.get("SLURM_JOB_NODELIST", os.environ.get("SLURM_NODELIST", "")))
    if host:
        return host
    raise RuntimeError("multi-node launch without MASTER_ADDR: set MASTER_ADDR to the host of rank 0")


def setup_distributed_environment() -> Dict[str, Any]:
    """Normalise the launch environment to RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR /
    MASTER_PORT (written to os.environ for torch.distributed's env:// rendezvous) and describe it:
    {'launcher': 'torchrun'|'mpiexec'|'single', rank, world_size, local_rank, master_addr,
    master_port}."""
    env = os.environ
    if all(v in env for v in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")):
        return {"launcher": "torchrun", "rank": int(env["RANK"]), "world_size": int(env["WORLD_SIZE"]),
                "local_rank": int(env.get("LOCAL_RANK", "0")), "master_addr": env["MASTER_ADDR"],
                "master_port": int(env["MASTER_PORT"])}
    if detect_mpi_environment():
        info = get_mpi_info()
        if info["rank"] is None or info["world_size"] is None:
            raise RuntimeError("Could not determine MPI rank and world size")
        addr = _master_addr(info)
        port = int(env.get("MASTER_PORT", DEFAULT_PORT))
        env.update(RANK=str(info["rank"]), WORLD_SIZE=str(info["world_size"]),
                   LOCAL_RANK=str(info["local_rank"]), MASTER_ADDR=addr, MASTER_PORT=str(port))
        return {"launcher": "mpiexec", "rank": info["rank"], "world_size": info["world_size"],
                "local_rank": info["local_rank"], "master_addr": addr, "master_port": port}
    return {"launcher": "single", "rank": 0, "world_size": 1, "local_rank": 0,
            "master_addr": LOOPBACK, "master_port": DEFAULT_PORT}


def get_device_for_rank(rank: Optional[int] = None) -> torch.device:
    """The CUDA device of a rank (rank modulo the visible devices; LOCAL_RANK when no rank is
    given and the launcher set it); the CPU device when there is no GPU, which only the host-side
    tests use."""
    if rank is None:
        if "LOCAL_RANK" in os.environ:
            rank = int(os.environ["LOCAL_RANK"])
        else:
            rank = dist.get_rank() if dist.is_initialized() else 0
    if torch.cuda.is_available():
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


def init_distributed_backend(backend: Optional[str] = None, timeout_seconds: int = 1800) -> bool:
    """Initialise the default process group from the launch environment. True on success, when
    already initialised, or for a single process (nothing to initialise); False when the backend
    fails to come up."""
    if dist.is_initialized():
        return True
    info = setup_distributed_environment()
    if info["world_size"] == 1:
        _say("single process: no process group")
        return True
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kwargs: Dict[str, Any] = {"backend": backend,
                              "timeout": datetime.timedelta(seconds=timeout_seconds)}
    if backend == "nccl":
        from .hybrid import high_priority_nccl_options
        device = get_device_for_rank(info["local_rank"])
        torch.cuda.set_device(device)
        kwargs.update(device_id=device, pg_options=high_priority_nccl_options())
    _say(f"{info['launcher']}: rank {info['rank']}/{info['world_size']} via "
         f"{info['master_addr']}:{info['master_port']} on {backend}")
    try:
        dist.init_process_group(**kwargs)
        return True
    except Exception as exc:  # noqa: BLE001 - the reference's contract is a boolean
        _say(f"{backend} initialisation failed: {exc}")
        return False


def cleanup_distributed() -> None:
    """Destroy the default process group if there is one."""
    if dist.is_initialized():
        dist.destroy_process_group()


def node_major_ring_order(world_size: int, local_size: int) -> List[List[int]]:
    """Ranks of each node in ring order for a launch of `world_size` ranks with `local_size`
    per node (ranks numbered node by node, as mpiexec, srun and torchrun do). Consecutive ring
    neighbours share a node's NVLink domain except for one hop per node that crosses the
    inter-node fabric; a hybrid setup puts the Ulysses all-to-all inside a node
    (`sp_ulysses_degree` = local_size) and the ring across nodes."""
    if local_size <= 0 or world_size % local_size:
        raise ValueError(f"world size {world_size} is not a multiple of ranks per node {local_size}")
    return [list(range(n * local_size, (n + 1) * local_size)) for n in range(world_size // local_size)]


def setup_mpi_distributed(backend: Optional[str] = None) -> Dict[str, Any]:
    """One call for a training script: normalise the environment, initialise the process group
    when there is more than one rank, pick the device. Returns {rank, world_size, local_rank,
    device, launcher, backend}; raises RuntimeError when the backend cannot be initialised."""
    info = setup_distributed_environment()
    if info["world_size"] > 1 and not init_distributed_backend(backend):
        raise RuntimeError("Failed to initialize distributed backend")
    return {"rank": info["rank"], "world_size": info["world_size"], "local_rank": info["local_rank"],
            "device": get_device_for_rank(info["local_rank"]), "launcher": info["launcher"],
            "backend": dist.get_backend() if dist.is_initialized() else None}
