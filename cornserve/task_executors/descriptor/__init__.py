from .base import LaunchSpec, TaskExecutionDescriptor  # noqa: F401
