from torchsso.optim.secondorder import SecondOrderOptimizer, DistributedSecondOrderOptimizer  # noqa: F401
from torchsso.optim.vi import VIOptimizer, DistributedVIOptimizer, VOGN  # noqa: F401
