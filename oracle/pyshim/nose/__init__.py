"""Stand-in for `nose` (not installed): the few names the reference's Python
tests import, mapped onto unittest."""
