"""Context: the handle every call takes (replaces the reference's rt::Device,
metal_pjrt/runtime/metal_runtime.h:276-450, for a CUDA caller)."""
import ctypes as C

from . import _lib


class Context:
    def __init__(self, device=0):
        handle = C.c_void_p()
        _lib.check(_lib.lib().b200_context_create(device, C.byref(handle)))
        self.handle = handle
        self.device = device

    def close(self):
        if self.handle:
            _lib.lib().b200_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def error(self):
        """Sticky status (0 = OK); folds in device-side reports."""
        return _lib.lib().b200_context_error(self.handle)

    def fail_launch_after(self, n):
        _lib.lib().b200_context_fail_launch_after(self.handle, n)

    @property
    def launch_count(self):
        return _lib.lib().b200_context_launch_count(self.handle)


_default = {}


def default_context(device=0):
    if device not in _default:
        _default[device] = Context(device)
    return _default[device]
