from torcheval.metrics import Metric  # noqa: F401
