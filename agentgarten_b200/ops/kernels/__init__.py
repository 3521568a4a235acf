"""Kernel entry points under their historical names (``wm.kernels.*``)."""
