from .barrier import barrier, barrier_test, wait_never
from .collectives import (all_gather, all_reduce, choose_all_reduce_algo, one_shot_all_gather,
                          one_shot_all_reduce, one_shot_reduce_scatter, reduce_scatter)
