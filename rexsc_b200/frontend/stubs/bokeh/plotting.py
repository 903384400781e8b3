from . import _absent

figure = _absent("plotting.figure")
