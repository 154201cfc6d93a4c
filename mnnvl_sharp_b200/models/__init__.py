"""Layers that consume the collectives: tensor-parallel FP8 linear / FFN, data-parallel gradient averaging."""
from .dp_reducer import GradientAllReducer  # noqa: F401
from .tp_linear import RowParallelLinearFP8, TensorParallelFFN, TensorParallelFFNDown  # noqa: F401
