"""CPU oracle for the docc library-node hot path. Test infrastructure only."""
from .oracle import *  # noqa: F401,F403
