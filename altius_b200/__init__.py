"""session_cuda: a B200-native execution backend behind altius's session API."""
from . import ir  # noqa: F401
