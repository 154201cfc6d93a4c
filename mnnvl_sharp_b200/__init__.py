"""B200-native NVLink-SHARP (multimem) all-reduce framework.

Layers: `utils` (host numerics, oracle, rack inventory), `parallel` (control plane, symmetric
memory, communicator), `ops` (all-reduce and fused GEMM+all-reduce on symmetric tensors),
`models` (tensor-parallel layers built on the ops), `cli` (launcher, preflight, sweeps).
"""
__version__ = "0.1.0"
