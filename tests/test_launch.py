"""Process bootstrap (torchrun / mpiexec / srun) — host logic only; counterpart of the
reference's sp_aurora/mpi_utils.py:16-320."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

LAUNCH_VARS = [
    "RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT",
    "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK",
    "OMPI_COMM_WORLD_LOCAL_SIZE", "PMI_RANK", "PMI_SIZE", "MPI_LOCALRANKID", "MPI_LOCALNRANKS",
    "PMIX_RANK", "PMIX_SIZE", "PMIX_LOCAL_RANK", "PMIX_LOCAL_SIZE", "MV2_COMM_WORLD_RANK",
    "MV2_COMM_WORLD_SIZE", "MV2_COMM_WORLD_LOCAL_RANK", "MV2_COMM_WORLD_LOCAL_SIZE", "MPI_RANK",
    "MPI_SIZE", "MPI_WORLD_SIZE", "MPI_LOCAL_RANK", "MPI_LOCAL_SIZE", "SLURM_PROCID", "SLURM_NTASKS",
    "SLURM_LOCALID", "SLURM_NTASKS_PER_NODE", "SLURM_JOB_NODELIST", "SLURM_NODELIST",
    "SLURM_LAUNCH_NODE_IPADDR",
]


@pytest.fixture
def clean_env(monkeypatch):
    for v in LAUNCH_VARS:
        monkeypatch.delenv(v, raising=False)
    return monkeypatch


def test_single_process(clean_env):
    from sp_aurora_b200 import mpi_utils as mu
    assert not mu.detect_mpi_environment()
    assert mu.get_mpi_info() == {"rank": None, "world_size": None, "local_rank": None, "local_size": None}
    info = mu.setup_distributed_environment()
    assert info == {"launcher": "single", "rank": 0, "world_size": 1, "local_rank": 0,
                    "master_addr": "127.0.0.1", "master_port": 29500}
    assert mu.init_distributed_backend() is True and not dist.is_initialized()
    res = mu.setup_mpi_distributed()
    assert res["world_size"] == 1 and res["backend"] is None and res["launcher"] == "single"


def test_torchrun_environment_is_taken_as_is(clean_env):
    from sp_aurora_b200 import mpi_utils as mu
    for k, v in dict(RANK="3", WORLD_SIZE="8", LOCAL_RANK="3", MASTER_ADDR="127.0.0.1",
                     MASTER_PORT="29511").items():
        clean_env.setenv(k, v)
    clean_env.setenv("OMPI_COMM_WORLD_RANK", "5")       # torchrun's variables win
    info = mu.setup_distributed_environment()
    assert info == {"launcher": "torchrun", "rank": 3, "world_size": 8, "local_rank": 3,
                    "master_addr": "127.0.0.1", "master_port": 29511}


@pytest.mark.parametrize("family", [
    dict(OMPI_COMM_WORLD_RANK="5", OMPI_COMM_WORLD_SIZE="8", OMPI_COMM_WORLD_LOCAL_RANK="5",
         OMPI_COMM_WORLD_LOCAL_SIZE="8"),
    dict(PMI_RANK="5", PMI_SIZE="8", MPI_LOCALRANKID="5", MPI_LOCALNRANKS="8"),
    dict(PMIX_RANK="5", PMIX_SIZE="8", PMIX_LOCAL_RANK="5", PMIX_LOCAL_SIZE="8"),
    dict(MV2_COMM_WORLD_RANK="5", MV2_COMM_WORLD_SIZE="8", MV2_COMM_WORLD_LOCAL_RANK="5",
         MV2_COMM_WORLD_LOCAL_SIZE="8"),
    dict(MPI_RANK="5", MPI_WORLD_SIZE="8", MPI_LOCAL_RANK="5", MPI_LOCAL_SIZE="8"),
    dict(SLURM_PROCID="5", SLURM_NTASKS="8", SLURM_LOCALID="5", SLURM_NTASKS_PER_NODE="8(x1)"),
])
def test_mpi_families_single_node(clean_env, family):
    from sp_aurora_b200 import mpi_utils as mu
    for k, v in family.items():
        clean_env.setenv(k, v)
    assert mu.detect_mpi_environment()
    assert mu.get_mpi_info() == {"rank": 5, "world_size": 8, "local_rank": 5, "local_size": 8}
    info = mu.setup_distributed_environment()
    assert info == {"launcher": "mpiexec", "rank": 5, "world_size": 8, "local_rank": 5,
                    "master_addr": "127.0.0.1", "master_port": 29500}
    # the env:// rendezvous variables are in place for torch.distributed
    assert (os.environ["RANK"], os.environ["WORLD_SIZE"], os.environ["LOCAL_RANK"],
            os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"]) == ("5", "8", "5", "127.0.0.1", "29500")


def test_multi_node_needs_an_address(clean_env):
    from sp_aurora_b200 import mpi_utils as mu
    for k, v in dict(OMPI_COMM_WORLD_RANK="9", OMPI_COMM_WORLD_SIZE="16", OMPI_COMM_WORLD_LOCAL_RANK="1",
                     OMPI_COMM_WORLD_LOCAL_SIZE="8").items():
        clean_env.setenv(k, v)
    with pytest.raises(RuntimeError, match="MASTER_ADDR"):
        mu.setup_distributed_environment()
    clean_env.setenv("MASTER_ADDR", "10.0.0.7")
    clean_env.setenv("MASTER_PORT", "23456")
    info = mu.setup_distributed_environment()
    assert (info["master_addr"], info["master_port"], info["local_rank"]) == ("10.0.0.7", 23456, 1)


def test_slurm_node_list(clean_env):
    from sp_aurora_b200 import mpi_utils as mu
    assert mu.first_slurm_host("node[03-05,9],x1") == "node03"
    assert mu.first_slurm_host("gpu7") == "gpu7"
    assert mu.first_slurm_host("a[1,4]") == "a1"
    assert mu.first_slurm_host("") is None
    for k, v in dict(SLURM_PROCID="8", SLURM_NTASKS="16", SLURM_LOCALID="0", SLURM_NTASKS_PER_NODE="8(x2)",
                     SLURM_JOB_NODELIST="b200-[11-12]").items():
        clean_env.setenv(k, v)
    assert mu.setup_distributed_environment()["master_addr"] == "b200-11"


def test_incomplete_mpi_environment_raises(clean_env):
    from sp_aurora_b200 import mpi_utils as mu
    clean_env.setenv("PMI_RANK", "0")
    with pytest.raises(RuntimeError, match="rank and world size"):
        mu.setup_distributed_environment()


def test_ring_order_and_device(clean_env):
    from sp_aurora_b200 import mpi_utils as mu
    assert mu.node_major_ring_order(16, 8) == [list(range(8)), list(range(8, 16))]
    with pytest.raises(ValueError):
        mu.node_major_ring_order(12, 8)
    if not torch.cuda.is_available():
        assert mu.get_device_for_rank(3) == torch.device("cpu")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _mpi_worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    for v in LAUNCH_VARS:
        os.environ.pop(v, None)
    # what `mpiexec -n 2` (Open MPI) gives each process, plus the port the test picked
    os.environ.update(OMPI_COMM_WORLD_RANK=str(rank), OMPI_COMM_WORLD_SIZE=str(world),
                      OMPI_COMM_WORLD_LOCAL_RANK=str(rank), OMPI_COMM_WORLD_LOCAL_SIZE=str(world),
                      MASTER_PORT=str(port))
    import sp_aurora_b200 as spa
    res = spa.setup_mpi_distributed(backend="gloo")
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t)
    again = spa.init_distributed_backend()          # already initialised: True, nothing done
    ret[rank] = (res["rank"], res["world_size"], res["local_rank"], res["launcher"], res["backend"],
                 str(res["device"]), float(t.item()), again)
    spa.cleanup_distributed()
    ret[f"clean{rank}"] = not dist.is_initialized()


def test_mpi_launch_initialises_gloo_group():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_mpi_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        rank, world, lrank, launcher, backend, device, total, again = ret[r]
        assert (rank, world, lrank, launcher, backend) == (r, 2, r, "mpiexec", "gloo")
        assert total == 3.0 and again is True and ret[f"clean{r}"]
