from .descriptor_registry import DESCRIPTOR_REGISTRY, TaskExecutionDescriptorRegistry, register_descriptor  # noqa: F401
from .task_class_registry import TASK_CLASS_REGISTRY, TaskClassRegistry, register_task  # noqa: F401
