"""linghe_b200 -- sm_100a (B200) CUDA implementation of the fused RMSNorm / SwiGLU +
FP8 e4m3 blockwise-quantisation path of inclusionAI/linghe, behind that library's own
Python entry points (same names, signatures, tensor and scale layouts).

Layout of the package:
  csrc/      hand-written CUDA kernels and the C ABI (include/linghe_b200.h)
  _lib.py    ctypes binding of the C ABI
  utils/     norm.py, silu.py   -- mirrors linghe/utils/{norm,silu}.py
  quant/     block.py, group.py -- mirrors linghe/quant/{block,group}.py
  facade/    norm.py, silu.py   -- mirrors linghe/facade/{norm,silu}.py (autograd glue)
  tools/     check.py, benchmark.py
There is no CPU path and no fallback: every entry point needs the built CUDA library
and an sm_100 device.
"""

__version__ = "0.1.0"
