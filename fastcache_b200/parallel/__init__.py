from .tp import (init_tensor_parallel, cleanup_tensor_parallel, get_tp_size, get_tp_rank, get_tp_group,
                 is_tp_initialized, tp_all_reduce, tp_all_gather, tp_broadcast, tp_barrier,
                 get_tensor_model_parallel_world_size, get_tensor_model_parallel_rank)  # noqa: F401
