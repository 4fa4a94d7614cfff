"""`krn.runtime.host`: the names the Python program AROUND the kernels uses, under the module path the reference gives
them (src/krn/runtime/host.py) — `host.Device.current()` is the B200 device, `host.Stream` / `host.Event` its in-order
queues and awaitable points, `host.Graph` a recorded launch sequence, `host.Settings` the settings snapshot. Only what
the tile-product and attention path needs is present: pipelines, precision ladders, compile options and the machine
inventory of the reference's module belong to subsystems this package does not rebuild."""

from krn_b200.runtime.api import Bound, Configured, Device, Event, Graph, Launcher, Stream
from krn_b200.runtime.device import default_device
from krn_b200.runtime.settings import Settings

__all__ = ["Bound", "Configured", "Device", "Event", "Graph", "Launcher", "Settings", "Stream", "default_device"]
