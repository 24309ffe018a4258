"""B200-native K-FAC curvature path behind the PyTorch-SSO API.

Same names as the reference package (torchsso/__init__.py:1-18): ``torchsso.optim``,
``torchsso.utils`` and the curvature classes that the optimizers look up by name.
The Hessian curvatures of the reference (marked work-in-progress there) are not provided.
"""
from torchsso.curv.curvature import Curvature, DiagCurvature, KronCurvature  # noqa: F401
from torchsso.curv.layers import (  # noqa: F401
    Fisher, CovLinear, DiagCovLinear, KronCovLinear, CovConv2d, DiagCovConv2d, KronCovConv2d,
    CovBatchNorm1d, DiagCovBatchNorm1d, CovBatchNorm2d, DiagCovBatchNorm2d,
    DiagFisherLinear, KronFisherLinear, DiagFisherConv2d, KronFisherConv2d, DiagFisherBatchNorm2d)
from torchsso.curv.fisher import get_closure_for_fisher  # noqa: F401
from torchsso.curv.pool import FactorPool  # noqa: F401
from torchsso import utils  # noqa: F401
from torchsso import optim  # noqa: F401

__version__ = '0.1.1+b200'
