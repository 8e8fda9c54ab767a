from .schema import SidecarConfig  # noqa: F401
