"""CPU oracle package (TEST INFRASTRUCTURE).  Importable only by tests, the smoke check and the
benchmark's cpu_baseline / reference legs; the product package never imports it."""
from . import oracle_np  # noqa: F401
from .build_oracle import build_oracle, load_oracle  # noqa: F401
from .oracle_c import OracleC  # noqa: F401
