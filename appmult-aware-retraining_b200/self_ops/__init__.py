"""`self_ops` - drop-in for the reference package of the same name (self_ops/__init__.py:1):
`import self_ops; self_ops.init_lookup_tables(...); self_ops.approx_conv2d_op(...)`."""
from .ops_py import *  # noqa: F401,F403
from .ops_py import __all__  # noqa: F401
