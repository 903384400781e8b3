"""Import stand-in for the ``bokeh`` plotting package.

The reference's ``utils.py`` imports bokeh at module level (utils.py:7-9) for its unused ``ResultsLog`` plots.
Machines that run the SC arithmetic rarely have bokeh; this package lets the unchanged module import.  Every entry
point raises when it is actually called.  The directory that holds it is appended to the END of ``sys.path``, so a
real bokeh installation always wins."""


def _absent(name):
    def fn(*args, **kwargs):
        raise RuntimeError(f"bokeh.{name}: bokeh is not installed; this is an import stand-in only")
    fn.__name__ = name
    return fn
