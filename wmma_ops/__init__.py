"""Drop-in module name: ``import wmma_ops`` resolves to the B200 implementation.

The reference builds an extension module called ``wmma_ops`` (setup.py:20-22); callers that
do ``import wmma_ops; wmma_ops.matmul(A, B)`` keep working unchanged.
"""
from wmma_ops_b200 import *  # noqa: F401,F403
from wmma_ops_b200 import __version__  # noqa: F401
