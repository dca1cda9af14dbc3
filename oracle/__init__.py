"""CPU oracle (test infrastructure): ctypes binding of oracle/liboracle.so. See oracle/oracle.c."""
from .oracle import *  # noqa: F401,F403
