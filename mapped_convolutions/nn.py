from mappedconvolutions_b200.nn import *  # noqa: F401,F403
from mappedconvolutions_b200.nn import __all__  # noqa: F401
