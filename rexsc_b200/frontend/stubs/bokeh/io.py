from . import _absent

output_file = _absent("io.output_file")
save = _absent("io.save")
show = _absent("io.show")
