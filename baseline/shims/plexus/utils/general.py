def print_axonn_timer_data(*a, **kw):
    pass
