"""Helper shared by the two config generators (gemm/gemm_configs.py and
flashattention/flash_configs.py)."""


class write_if_changed:
    """open(path, "w") that leaves the file (and its mtime) alone when the content is
    unchanged, so a rebuild is triggered only by a real change of the config list."""

    def __init__(self, path):
        self.path = path
        self.parts = []

    def __enter__(self):
        return self

    def write(self, text):
        self.parts.append(text)

    def __exit__(self, *exc):
        text = "".join(self.parts)
        try:
            with open(self.path, "r", encoding="utf-8") as f:
                if f.read() == text:
                    return False
        except OSError:
            pass
        with open(self.path, "w", encoding="utf-8") as f:
            f.write(text)
        return False
