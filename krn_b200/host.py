"""`krn.host`: short spelling of `krn.runtime.host` (`from krn import host`, src/krn/__init__.py)."""

from krn_b200.runtime.host import *  # noqa: F401,F403
from krn_b200.runtime.host import __all__  # noqa: F401
