from .tp_mlp import TensorParallelMLP
