from . import _absent

column = _absent("layouts.column")
