from torchsso.utils.logger import Logger  # noqa: F401
from torchsso.utils.linalg import inv, cholesky  # noqa: F401
from torchsso.utils.accumulator import TensorAccumulator  # noqa: F401
from torchsso.utils.communicator import KFACCommunicator, create_communicator, assign_owners  # noqa: F401
from torchsso.utils.graphs import GraphedClosure  # noqa: F401
from torchsso.utils.prefetch import BatchPrefetcher  # noqa: F401
from torchsso._native import set_curvature_stream, curvature_stream_enabled  # noqa: F401
from torchsso._native import set_factor_batching, factor_batching_enabled  # noqa: F401
