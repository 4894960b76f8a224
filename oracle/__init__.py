"""CPU oracle for the conv2d hot path.  TEST INFRASTRUCTURE, not product code.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this package; nothing under ``flagdnn_b200/`` does.
"""
from .conv_oracle import (  # noqa: F401
    build,
    conv2d_loops,
    conv2d_torch_cpu,
    conv_out_dim,
    normalize_padding,
)
