"""Capture of tile kernels (source → typed IR), launch-geometry inference and the recogniser that maps the
captured patterns onto the prebuilt sm_100a kernels."""
