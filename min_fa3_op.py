"""Drop-in module name of the reference API: ``import min_fa3_op`` resolves to the B200
implementation in ``min_fa3_demo_b200.min_fa3_op``."""
from min_fa3_demo_b200.min_fa3_op import *  # noqa: F401,F403
from min_fa3_demo_b200.min_fa3_op import __all__, _debug_resolve_launch_grid_shape  # noqa: F401
