from .linalg import matrix_multiply  # noqa: F401
