from .linalg import MatrixMultiply  # noqa: F401
