"""CPU oracle for the B200 tile-product / attention kernels — TEST INFRASTRUCTURE, not product code.

Only `tests/`, `__graft_entry__.smoke()` and the CPU-baseline legs of `bench.py` may import this package.
See `oracle/krn_oracle.c` for what is restated and which parts are pinned against the reference's own
known-answer tests.
"""

from oracle.oracle import *  # noqa: F401,F403
