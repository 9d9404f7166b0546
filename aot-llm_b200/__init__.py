"""aot-llm_b200: a B200 (sm_100a) implementation of aot-llm's quantized forward-pass
hot path behind the reference's kernel surface.

The directory name carries a hyphen, so load it with `import_package()` from
`__graft_entry__` (or importlib) under the module name `aot_llm_b200`.
"""
from . import build, lib, gpu, model, ranks, tp, session, gguf  # noqa: F401
from .gpu import Context, Gpu, DeviceBuffer  # noqa: F401
from .lib import AotCudaError  # noqa: F401
