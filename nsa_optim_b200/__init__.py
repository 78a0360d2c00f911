"""nsa_optim_b200: a Blackwell (B200, sm_100a) training framework for hybrid
Mamba-2 / Gated DeltaNet / (native sparse) attention language models with low-bit optimizers.

Layout: ``config`` (sizes, flags, grid), ``models`` (four families + factories), ``ops``
(dispatch, PyTorch implementations, sm_100a CUDA kernels), ``optimizers``, ``parallel``
(sharded-parameter runtime and the NVLink peer-memory kernels), ``data``, ``checkpoint``,
``train`` (CLI), ``profiling``, ``benchmarks``, ``analysis``.
"""
__version__ = "0.1.0"
