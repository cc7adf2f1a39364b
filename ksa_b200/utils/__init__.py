from .common import Timer, dist_reduce_dict, get_rank, get_world_size, print_rank_0, set_random_seed, to_cuda
from .logger import get_logger, setup_logging

__all__ = ["Timer", "dist_reduce_dict", "get_rank", "get_world_size", "print_rank_0", "set_random_seed", "to_cuda",
           "get_logger", "setup_logging"]
