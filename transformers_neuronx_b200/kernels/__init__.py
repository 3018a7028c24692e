from . import build, ops
from .build import KernelBuildError, build_all, build_many
from .ops import KernelError
from .profile import KernelProfile, kernel_profile
