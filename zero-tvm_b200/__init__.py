"""ztvm-b200: hand-written CUDA (sm_100a) kernels for Zero-TVM's int4 / int3 group-quantised
dequant-matmul family, behind a C ABI (include/ztvm_b200.h).

`capi`     ctypes binding of the C ABI (the same surface a Node-API addon binds)
`backend`  host-side mirror of the engine's matmul dispatch surface (entry names, PODArgs, bind
           groups, grids) on top of `capi`
`synth`    seeded synthetic tensors in the kernels' layouts
`build`    nvcc build of libztvm_b200.so
`recorder` a decode step's dispatch sequence captured once into a CUDA graph
`ingest`   MLX safetensors records -> the buffers the kernels bind (host side, numpy)

There is no CPU implementation: importing is cheap, but creating a Context without the built
library or without a B200 raises.
"""
from . import capi, synth  # noqa: F401
from .capi import Context, MmDesc, MoeDesc, MoeEpLayout, MoeEpRows, MoeFfnEpArgs, ZtvmError  # noqa: F401
from . import backend  # noqa: F401
from . import sharded  # noqa: F401,E402
from . import build  # noqa: F401,E402
from . import ingest  # noqa: F401,E402
from . import recorder  # noqa: F401,E402
