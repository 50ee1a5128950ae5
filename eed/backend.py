"""``eed.backend`` as the reference's scripts import it, served by fastgate_b200."""
from fastgate_b200.ops import *  # noqa: F401,F403
