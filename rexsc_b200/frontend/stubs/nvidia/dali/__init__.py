"""Import stand-in for NVIDIA DALI (``nvidia.dali``).

The reference's ``utils.py`` imports DALI at module level (utils.py:14-17) for its ImageNet input pipeline
(utils.py:238-290).  Data loading is outside the SC arithmetic path and synthetic inputs are used instead, so only
the import has to succeed: ``pipeline_def`` returns a function that raises when a pipeline is requested.
``nvidia`` itself is left a namespace package (no ``__init__``) so the CUDA wheels that install under the same
top-level name keep working, and the directory is appended to the END of ``sys.path``."""


def pipeline_def(fn=None, **kwargs):
    def build(*a, **k):
        raise RuntimeError("nvidia.dali is not installed; this is an import stand-in only")
    if fn is None:
        return lambda f: build
    return build
