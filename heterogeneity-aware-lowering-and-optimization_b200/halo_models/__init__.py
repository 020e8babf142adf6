"""Model descriptions that follow the emission rules of HALO's generic C++ code generator
(Conv with a null bias followed by a per-channel Add, residual Add then Relu, ReduceMean for the
global pool, Gemm for every matmul) and drive any ODLA platform library through ``odla.Graph``."""
from . import bert, mnist, resnet50, yolov3  # noqa: F401
