from .comm import Communicator  # noqa: F401
