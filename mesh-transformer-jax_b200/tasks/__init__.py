from .eval_harness import EvalHarnessAdaptor  # noqa: F401
