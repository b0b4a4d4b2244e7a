from pfeife_b200.runtime.local import LocalReducer, LocalRunner  # noqa: F401
