"""Stand-in for ``nvidia.dali.fn``: any operator lookup raises."""


def __getattr__(name):
    raise RuntimeError(f"nvidia.dali.fn.{name}: DALI is not installed; this is an import stand-in only")
