"""One CPU rank of a job that meets through a shared file instead of a TCP store (run by
tests/test_fault_tolerance.py::test_file_rendezvous)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    for k in ("MASTER_ADDR", "MASTER_PORT"):
        os.environ.pop(k, None)
    os.environ["ITB_RDZV_FILE"] = path
    from infinitrain_b200.parallel import global_env as genv
    from infinitrain_b200.parallel.process_group import ProcessGroupFactory, ReduceOpType

    genv.InitAllEnv(world_size=world, rank=rank)
    pg = ProcessGroupFactory.Instance().Init(backend="gloo", timeout_s=60).GetDefaultProcessGroup()
    t = torch.full((3,), float(rank + 1))
    pg.AllReduce(t, ReduceOpType.kSum)
    assert t.tolist() == [float(sum(range(1, world + 1)))] * 3, t
    print(f"rank {rank} ok")


if __name__ == "__main__":
    main()
