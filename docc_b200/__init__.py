"""docc_b200 — B200 (sm_100a) kernels for the library nodes docc's CUDA target executes.

``docc_b200.ops``       array-level calls into the C ABI (numpy = host pointers, torch CUDA = device pointers)
``docc_b200.nodes``     library-node descriptions and dispatch, mirroring docc's node API
``docc_b200.python``    ``@native`` front end
``docc_b200.torch``     ``torch.compile(backend="docc")`` front end
"""
from . import ops  # noqa: F401
from ._lib import DoccB200Error  # noqa: F401

__version__ = "0.1.0"
