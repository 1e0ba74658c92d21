"""`utils_ccm.module_ccm` of the reference: the older module name for the same compressors."""
from .module_ccm_v11 import *  # noqa: F401,F403
