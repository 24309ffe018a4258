from torchsso.curv.curvature import Curvature, DiagCurvature, KronCurvature  # noqa: F401
from torchsso.curv.pool import FactorPool  # noqa: F401
from torchsso.curv.layers import *  # noqa: F401,F403
from torchsso.curv.fisher import get_closure_for_fisher  # noqa: F401
