from .sageconv import DistSAGEConvGrad  # noqa: F401
