"""Process-level helpers: device selection, seeding and process-group start-up.

Counterparts in hpcaitech/Elixir: ``elixir/cuda.py:10-12`` (gpu_device), ``elixir/utils.py:26-56``
(seed_all, init_distributed).
"""
import os
import random

import torch
import torch.distributed as dist


def gpu_device() -> torch.device:
    """The CUDA device of this process."""
    if not torch.cuda.is_available():
        raise RuntimeError('elixir_b200 needs a CUDA device')
    return torch.device('cuda', torch.cuda.current_device())


def seed_all(seed: int, cuda_deterministic: bool = False):
    random.seed(seed)
    try:
        import numpy as np
        np.random.seed(seed)
    except ImportError:
        pass
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
        torch.backends.cudnn.deterministic = bool(cuda_deterministic)
        torch.backends.cudnn.benchmark = not cuda_deterministic


def init_distributed(backend: str = None):
    """Join the job described by RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT: one process
    per GPU, NCCL over NVLink when CUDA is present (gloo otherwise, for host-logic tests)."""
    rank = int(os.environ['RANK'])
    local_rank = int(os.environ.get('LOCAL_RANK', rank))
    world_size = int(os.environ['WORLD_SIZE'])
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29512')
    if backend is None:
        backend = 'nccl' if torch.cuda.is_available() else 'gloo'
    if backend == 'nccl':
        torch.cuda.set_device(local_rank)
        dist.init_process_group(backend, rank=rank, world_size=world_size,
                                device_id=torch.device('cuda', local_rank))
    else:
        dist.init_process_group(backend, rank=rank, world_size=world_size)
    seed_all(1024)
    return rank, world_size


def print_rank_0(*args, **kwargs):
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(*args, **kwargs)
