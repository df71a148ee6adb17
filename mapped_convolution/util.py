from mappedconvolutions_b200.util import *  # noqa: F401,F403
from mappedconvolutions_b200.util import __all__  # noqa: F401
