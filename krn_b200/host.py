"""`krn.host`: where kernels run (src/krn/runtime/host.py). `host.Device.current()` is the B200 device."""

from krn_b200.runtime.api import Bound, Device, Event, Graph, Launcher, Stream

__all__ = ["Bound", "Device", "Event", "Graph", "Launcher", "Stream"]
