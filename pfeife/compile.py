from pfeife_b200.compile import WrapperModule, compile_module  # noqa: F401
