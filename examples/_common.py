"""Set-up shared by the example scripts: one process per GPU under torchrun, or a single process."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def init(heap_size=1 << 30):
    """Initialise torch.distributed (nccl on GPUs, gloo otherwise) and return an Iris context."""
    import iris_b200 as iris

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    if torch.cuda.is_available():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    return iris.iris(heap_size)


def finish(ctx):
    ctx.barrier()
    dist.destroy_process_group()
