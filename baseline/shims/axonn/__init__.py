"""Minimal stand-in of AxoNN for running the reference without the library: no-op region timers, no group factory
(the reference is driven with ``use_axonn=False`` so it builds its groups with ``torch.distributed.new_group``)."""


class _Timers:
    def start(self, *a):
        pass

    def stop(self, *a):
        pass

    def get_times(self):
        return {}, {}


class _Axonn:
    is_initialized = False
    enable_timers = False
    timers = _Timers()
    comm_handle = None

    def init(self, *a, **kw):
        self.is_initialized = True

    def get_timers(self):
        return self.timers


axonn = _Axonn()
