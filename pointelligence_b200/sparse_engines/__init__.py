from . import _dispatch_override, _seg_offs, ops, tig  # noqa: F401
from ._dispatch_override import current_mode, dispatch_mode, precision_mode  # noqa: F401
