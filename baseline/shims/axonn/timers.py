from . import _Timers as Timers  # noqa: F401
