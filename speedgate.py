"""``import speedgate`` (the module name in the reference's setup.py:30), served by fastgate_b200."""
from fastgate_b200.ops import *  # noqa: F401,F403
