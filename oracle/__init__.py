"""CPU oracle for the parity tests (a restatement of the altius reference
interpreter). Test infrastructure only: the CUDA session never imports it."""
from .interpreter import InterpreterSession, InterpreterSessionBuilder  # noqa: F401
