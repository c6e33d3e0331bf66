def build_regex_from_schema(*a, **k):
    raise RuntimeError("outlines is not installed")
