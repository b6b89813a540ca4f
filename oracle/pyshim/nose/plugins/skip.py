from unittest import SkipTest  # noqa: F401
