"""Request / response models of the gateway's REST API (wire-compatible with
python/cornserve/services/gateway/models.py:10-111)."""

from __future__ import annotations

from typing import Any, Literal

from pydantic import BaseModel, Field


class AppRegistrationRequest(BaseModel):
    source_code: str


class AppInvocationRequest(BaseModel):
    request_data: dict[str, Any]


class ScaleTaskRequest(BaseModel):
    """Positive ``num_gpus`` scales up, negative scales down."""

    task_id: str
    num_gpus: int


class RegistrationInitialResponse(BaseModel):
    type: Literal["initial"] = "initial"
    app_id: str
    task_names: list[str]


class RegistrationFinalResponse(BaseModel):
    type: Literal["final"] = "final"
    message: str


class RegistrationErrorResponse(BaseModel):
    type: Literal["error"] = "error"
    message: str


class RegistrationStatusEvent(BaseModel):
    event: RegistrationInitialResponse | RegistrationFinalResponse | RegistrationErrorResponse = Field(discriminator="type")


class TaskDefinitionPayload(BaseModel):
    source_b64: str
    task_class_name: str
    task_definition_name: str
    module_name: str
    is_unit_task: bool = True


class DescriptorDefinitionPayload(BaseModel):
    source_b64: str
    descriptor_class_name: str
    descriptor_definition_name: str
    module_name: str
    task_class_name: str
    is_default: bool = True


class TasksDeploymentRequest(BaseModel):
    task_definitions: list[TaskDefinitionPayload] = []
    descriptor_definitions: list[DescriptorDefinitionPayload] = []


class ProfileDeploymentPayload(BaseModel):
    task: dict[str, Any]
    num_gpus_to_profile: dict[str, dict[str, Any]]


class ProfilesDeploymentRequest(BaseModel):
    profiles: list[ProfileDeploymentPayload]


class ReconcileRequest(BaseModel):
    task_id: str
    target_load: float
