"""Stand-in for ``nvidia.dali.plugin.pytorch`` (imported at utils.py:17)."""


class LastBatchPolicy:
    FILL = "FILL"
    DROP = "DROP"
    PARTIAL = "PARTIAL"


class DALIClassificationIterator:
    def __init__(self, *args, **kwargs):
        raise RuntimeError("nvidia.dali is not installed; this is an import stand-in only")
