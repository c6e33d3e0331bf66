"""Import stand-in: grammar-constrained requests are not part of the benchmark."""


class RegexGuide:
    def __init__(self, *a, **k):
        raise RuntimeError("outlines is not installed")

    @classmethod
    def from_regex(cls, *a, **k):
        raise RuntimeError("outlines is not installed")
