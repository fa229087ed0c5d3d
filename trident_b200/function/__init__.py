from .function import *  # noqa: F401,F403
