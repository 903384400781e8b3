"""Stand-in for the ``nvidia_smi`` NVML binding that the reference's ``utils_own.get_device`` imports inside the
function (utils_own.py:28) to wait for an idle GPU.  Backed by ``pynvml`` when that is importable; it only ever
READS utilisation, no setting of any GPU is touched."""
try:
    from pynvml import (nvmlInit, nvmlDeviceGetCount, nvmlDeviceGetHandleByIndex,  # noqa: F401
                        nvmlDeviceGetUtilizationRates)
except Exception:  # pragma: no cover - no NVML on this machine
    def _absent(*args, **kwargs):
        raise RuntimeError("nvidia_smi: no NVML binding is installed; pick the device explicitly")

    nvmlInit = nvmlDeviceGetCount = nvmlDeviceGetHandleByIndex = nvmlDeviceGetUtilizationRates = _absent
