"""The task programming model: ``Task`` / ``UnitTask`` / ``Stream`` / ``TaskInvocation`` /
``TaskGraphDispatch`` / ``TaskContext``.

Same public surface and wire formats as the reference (python/cornserve/task/base.py:77-838):
a composite task's synchronous ``invoke`` is run twice per call, first in *record* mode, where every
unit-task invocation returns a structurally correct placeholder and is appended to a list, then, after
the list has been dispatched and the real outputs have come back, in *replay* mode, where the same
invocations return the real outputs in the same order.
"""

from __future__ import annotations

import asyncio
import enum
import inspect
import json
import os
import uuid
from abc import ABC, abstractmethod
from collections import defaultdict, deque
from collections.abc import AsyncIterator, Callable, Iterable
from contextlib import contextmanager
from contextvars import ContextVar
from typing import TYPE_CHECKING, Any, ClassVar, Generic, TypeVar, final, get_type_hints

from pydantic import BaseModel, ConfigDict, Field, model_serializer, model_validator

from ..constants import GATEWAY_URL, TASK_TIMEOUT_S
from ..logging import get_logger
from ..tracing import get_tracer

if TYPE_CHECKING:  # pragma: no cover
    import aiohttp

logger = get_logger(__name__)


def _trace_configs():
    from ..tracing import aiohttp_trace_configs

    return aiohttp_trace_configs()
tracer = get_tracer(__name__)

TASK_TIMEOUT = TASK_TIMEOUT_S

_http_client: "aiohttp.ClientSession | None" = None


def get_client() -> "aiohttp.ClientSession":
    """Process-wide aiohttp session used when a task is invoked outside the gateway."""
    import aiohttp

    global _http_client
    if _http_client is None or _http_client.closed:
        _http_client = aiohttp.ClientSession(trace_configs=_trace_configs(), timeout=aiohttp.ClientTimeout(total=TASK_TIMEOUT),
                                             connector=aiohttp.TCPConnector(limit=0))
    return _http_client


# The recorder of the top-level call that is currently running in this asyncio context.
task_context: ContextVar["TaskContext"] = ContextVar("task_context")
# Set by the gateway at start-up: its in-process unit-task manager (invocations then skip the HTTP hop).
task_manager_context: ContextVar[Any] = ContextVar("task_manager_context", default=None)
# The task whose ``post_init`` is running; tasks constructed meanwhile become its sub-tasks.
current_task_context: ContextVar["Task | None"] = ContextVar("current_task_context", default=None)


class TaskInput(BaseModel):
    """Base class of task inputs."""


class TaskOutput(BaseModel):
    """Base class of task outputs."""


InputT = TypeVar("InputT", bound=TaskInput)
OutputT = TypeVar("OutputT", bound=TaskOutput)
TransformT = TypeVar("TransformT", bound=TaskOutput)


def _generic_args(obj: BaseModel) -> tuple:
    meta = type(obj).__pydantic_generic_metadata__
    if meta["origin"] is None:
        raise ValueError("Generic type argument is missing.")
    return meta["args"]


class Stream(TaskOutput, Generic[OutputT]):
    """Handle on a streamed task output: an async iterator of ``OutputT`` parsed from JSON lines."""

    async_iterator: Any = Field(default=None, exclude=True)  # AsyncIterator[str | bytes]
    response: Any = Field(default=None, exclude=True)        # aiohttp response kept open while streaming

    _prev_type: type[TaskOutput] | None = None
    _transform_func: Callable[[Any], Any] | None = None

    model_config = ConfigDict(arbitrary_types_allowed=True, extra="forbid")

    @model_validator(mode="after")
    def _check_item_type(self):
        _ = self.item_type
        return self

    @property
    def item_type(self) -> type[OutputT]:
        (arg,) = _generic_args(self)
        if not (inspect.isclass(arg) and issubclass(arg, TaskOutput)):
            raise ValueError(f"Generic type argument {arg} is not a subclass of TaskOutput.")
        return arg

    def transform(self, transform_func: Callable[[OutputT], TransformT],
                  output_type: type[TaskOutput] | None = None) -> "Stream[TransformT]":
        """Re-type the stream: items are parsed as the old type and mapped through ``transform_func``.
        The iterator moves to the new stream; a stream can be transformed once."""
        if self._transform_func is not None:
            raise ValueError("Cannot transform a stream more than once.")
        try:
            ret = get_type_hints(transform_func).get("return")
        except Exception:
            ret = None
        ret = ret or output_type
        if ret is None:
            raise ValueError("Output type must be specified if the transform function has no return type hint.")
        if not (inspect.isclass(ret) and issubclass(ret, TaskOutput)):
            raise ValueError(f"Return type {ret} is not a subclass of TaskOutput.")
        new = Stream[ret](async_iterator=self.async_iterator, response=self.response)
        new._prev_type = self.item_type
        new._transform_func = transform_func
        self.async_iterator = None
        self.response = None
        return new  # type: ignore[return-value]

    async def get_next(self) -> str | bytes | None:
        """Next raw line, or ``None`` at the end (the HTTP response is closed then)."""
        if self.async_iterator is None:
            raise ValueError("Stream generator is not initialized.")
        try:
            return await anext(self.async_iterator)
        except StopAsyncIteration:
            if self.response is not None:
                try:
                    self.response.close()
                except Exception as e:  # pragma: no cover
                    logger.warning("Failed to close stream response: %s", e)
            self.response = None
            self.async_iterator = None
            return None

    def __aiter__(self):
        return self

    async def __anext__(self) -> OutputT:
        if self.async_iterator is None:
            raise ValueError("Stream generator is not initialized.")
        while True:
            line = await self.get_next()
            if line is None:
                raise StopAsyncIteration
            line = line.strip()
            if line:
                break
        if self._transform_func is not None:
            assert self._prev_type is not None
            return self._transform_func(self._prev_type.model_validate_json(line))
        return self.item_type.model_validate_json(line)

    async def aiter_raw(self):
        """Iterate over the raw, non-empty lines without parsing (pass-through relays use this)."""
        if self.async_iterator is None:
            raise ValueError("Stream generator is not initialized.")
        while (line := await self.get_next()) is not None:
            line = line.strip()
            if line:
                yield line


class Task(BaseModel, ABC, Generic[InputT, OutputT]):
    """Base of all tasks.  Tasks constructed inside ``post_init`` are registered as sub-tasks
    (attribute names ``__subtask_<n>__`` listed in ``subtask_attr_names``)."""

    id: str = Field(init=False, default_factory=lambda: uuid.uuid4().hex)
    subtask_attr_names: list[str] = Field(init=False, default_factory=list)

    model_config = ConfigDict(extra="allow")

    def post_init(self) -> None:
        """Construct sub-tasks here."""

    def model_post_init(self, context: Any, /) -> None:
        parent = current_task_context.get()
        if parent is not None:
            name = f"__subtask_{len(parent.subtask_attr_names)}__"
            setattr(parent, name, self)
            parent.subtask_attr_names.append(name)
        token = current_task_context.set(self)
        try:
            self.post_init()
        finally:
            current_task_context.reset(token)

    @abstractmethod
    def invoke(self, task_input: InputT) -> OutputT:
        """Synchronous description of the computation in terms of other tasks."""

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        fn = cls.__dict__.get("invoke", cls.invoke)
        if not inspect.isfunction(fn):
            raise TypeError(f"{cls.__name__}.invoke should be a function")
        if inspect.iscoroutinefunction(fn):
            raise TypeError(f"{cls.__name__}.invoke should not be an async function")

    async def __call__(self, task_input: InputT) -> OutputT:
        task_context.set(TaskContext())
        return await asyncio.create_task(self._call_impl(task_input))

    async def _call_impl(self, task_input: InputT) -> OutputT:
        ctx = task_context.get()
        with ctx.record():
            self.invoke(task_input)
        await ctx.dispatch_tasks_and_wait()
        with ctx.replay():
            return self.invoke(task_input)


def discover_unit_tasks(tasks: Iterable[Task]) -> list["UnitTask"]:
    """All unit tasks reachable from ``tasks`` (depth first, in construction order)."""
    found: list[UnitTask] = []
    for t in tasks:
        if isinstance(t, UnitTask):
            found.append(t)
        else:
            found.extend(discover_unit_tasks(getattr(t, a) for a in t.subtask_attr_names))
    return found


def _is_unit_task_parametrisation(base: type) -> bool:
    """True for ``UnitTask`` itself and for the proxy classes ``UnitTask[In, Out]`` pydantic creates."""
    if base is UnitTask:
        return True
    # look at the class's own attribute only: while a subclass is being created it still sees the
    # metadata of its parent through normal attribute inheritance
    meta = base.__dict__.get("__pydantic_generic_metadata__")
    return bool(meta) and meta.get("origin") is UnitTask


class UnitTask(Task, Generic[InputT, OutputT]):
    """A task executed by one kind of executor; the unit of deployment, sharing and scaling.

    ``root_unit_task_cls`` is the first class below ``UnitTask[...]`` in the inheritance chain: it selects
    the compatible execution descriptors and defines which fields take part in equivalence.
    """

    root_unit_task_cls: ClassVar[type["UnitTask"]]

    execution_descriptor_name: str | None = None

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        if _is_unit_task_parametrisation(cls):
            cls.root_unit_task_cls = UnitTask
            return
        root: type = UnitTask
        for anc in cls.mro():
            if anc is UnitTask or not isinstance(anc, type) or not issubclass(anc, UnitTask):
                continue
            if _is_unit_task_parametrisation(anc):
                continue
            if any(_is_unit_task_parametrisation(b) for b in anc.__bases__):
                root = anc
                break
        cls.root_unit_task_cls = root

    @property
    def execution_descriptor(self):
        """Descriptor instance bound to this task (looked up by root class and descriptor name).

        Built with ``model_construct``: the registered descriptor class may have been created from an
        uploaded copy of the task class, so class-identity validation would reject an equal task."""
        from ..services.task_registry.descriptor_registry import DESCRIPTOR_REGISTRY

        cls = DESCRIPTOR_REGISTRY.get(self.root_unit_task_cls, self.execution_descriptor_name)
        return cls.model_construct(task=self)

    def is_equivalent_to(self, other: object) -> bool:
        """Equivalent tasks share one deployment: same root class (by name), same descriptor class and
        equal values of every root-class field except ``id`` and fields marked ``skip_comparison``."""
        if not isinstance(other, UnitTask):
            return False
        a, b = self.root_unit_task_cls, other.root_unit_task_cls
        if a is not b and a.__name__ != b.__name__:
            return False
        if type(self.execution_descriptor).__name__ != type(other.execution_descriptor).__name__:
            return False
        for name, info in a.model_fields.items():
            if name == "id":
                continue
            extra = info.json_schema_extra
            if isinstance(extra, dict) and extra.get("skip_comparison"):
                continue
            try:
                if getattr(self, name) != getattr(other, name):
                    return False
            except AttributeError:
                return False
        return True

    @abstractmethod
    def make_record_output(self, task_input: InputT) -> OutputT:
        """Placeholder output with the right structure (list lengths, forwards) for record mode."""

    def validate_input(self, task_input: InputT) -> None:
        """Hook called in record mode before the invocation is recorded."""

    @final
    def invoke(self, task_input: InputT) -> OutputT:
        ctx = task_context.get()
        if ctx.is_recording:
            self.validate_input(task_input)
            out = self.make_record_output(task_input)
            ctx.record_invocation(self, task_input, out)
            return out
        if ctx.is_replaying:
            return ctx.replay_invocation(self)  # type: ignore[return-value]
        raise AssertionError("Task context is neither in recording nor replay mode.")

    def make_name(self) -> str:
        return type(self).__name__.lower()


def _unit_task_classes(class_name: str):
    from ..services.task_registry.task_class_registry import TASK_CLASS_REGISTRY

    return TASK_CLASS_REGISTRY.get_unit_task(class_name)


class TaskInvocation(BaseModel, Generic[InputT, OutputT]):
    """One recorded unit-task call.  Serialised as ``{"class_name", "body": {"task", "task_input",
    "task_output"}}`` with JSON strings in the body; classes are resolved by name on the way back."""

    task: UnitTask
    task_input: TaskInput
    task_output: TaskOutput

    model_config = ConfigDict(arbitrary_types_allowed=True)

    @model_serializer()
    def _dump(self) -> dict[str, Any]:
        return {
            "class_name": type(self.task).__name__,
            "body": {
                "task": self.task.model_dump_json(),
                "task_input": self.task_input.model_dump_json(),
                "task_output": self.task_output.model_dump_json(),
            },
        }

    @model_validator(mode="before")
    @classmethod
    def _load(cls, data: Any):
        if not isinstance(data, dict) or "class_name" not in data:
            return data
        task_cls, in_cls, out_cls = _unit_task_classes(data["class_name"])
        body = data["body"]
        return {
            "task": task_cls.model_validate_json(body["task"]),
            "task_input": in_cls.model_validate_json(body["task_input"]),
            "task_output": out_cls.model_validate_json(body["task_output"]),
        }


class TaskGraphDispatch(BaseModel):
    """Payload sent to the task dispatcher.  Only the last invocation may produce a ``Stream``."""

    invocations: list[TaskInvocation]
    is_streaming: bool = False

    def model_post_init(self, context: Any, /) -> None:
        if not self.invocations:
            raise ValueError("Task graph must have at least one invocation.")
        if any(isinstance(i.task_output, Stream) for i in self.invocations[:-1]):
            raise ValueError("Only the last task invocation can have a stream output.")
        self.is_streaming = isinstance(self.invocations[-1].task_output, Stream)

    async def dispatch(self, url: str, client: "aiohttp.ClientSession") -> list[Any]:
        """POST the graph.  Non-streaming: the reply is the JSON list of outputs.  Streaming: line 1 is
        that list, the following lines are the chunks of the last invocation's stream."""
        import aiohttp

        with tracer.start_as_current_span("TaskGraphDispatch.dispatch"):
            try:
                if not self.is_streaming:
                    async with client.post(url, json=self.model_dump()) as resp:
                        resp.raise_for_status()
                        outputs = await resp.json()
                else:
                    resp = await client.post(url, json=self.model_dump())
                    resp.raise_for_status()
                    lines = _iter_lines(resp.content.iter_chunked(1 << 20))
                    try:
                        first = await anext(lines)
                    except StopAsyncIteration:
                        raise RuntimeError("Received incomplete response from the server.") from None
                    outputs = json.loads(first.strip())
                    outputs[-1]["async_iterator"] = lines
                    outputs[-1]["response"] = resp
                    type(self.invocations[-1].task_output).model_validate(outputs[-1])
            except aiohttp.ClientResponseError as e:
                raise RuntimeError(f"Received error response from {url}.") from e
            except aiohttp.ClientError as e:
                raise RuntimeError(f"Failed to send dispatch request to {url}.") from e
        if not isinstance(outputs, list):
            raise RuntimeError(f"Expected a list of task outputs, but got {type(outputs)}.")
        return outputs


async def _iter_lines(chunks: AsyncIterator[bytes]) -> AsyncIterator[bytes]:
    """Split a byte stream into lines without a per-line size limit (audio chunks can be large)."""
    pending = b""
    async for chunk in chunks:
        pending += chunk
        *lines, pending = pending.split(b"\n")
        for line in lines:
            yield line
    if pending:
        yield pending


class _Mode(enum.Enum):
    IDLE = 0
    RECORD = 1
    REPLAY = 2


class TaskContext:
    """Recorder of one top-level task call."""

    def __init__(self) -> None:
        self.invocations: list[TaskInvocation] = []
        self.task_outputs: dict[str, deque[TaskOutput]] = defaultdict(deque)
        self._mode = _Mode.IDLE

    @property
    def is_recording(self) -> bool:
        return self._mode is _Mode.RECORD

    @property
    def is_replaying(self) -> bool:
        return self._mode is _Mode.REPLAY

    @contextmanager
    def _enter(self, mode: _Mode):
        if self._mode is mode:
            raise RuntimeError(f"Task context is already in {mode.name.lower()} mode.")
        if self._mode is not _Mode.IDLE:
            raise RuntimeError(f"Cannot enter {mode.name.lower()} mode while in {self._mode.name.lower()} mode.")
        self._mode = mode
        try:
            yield
        finally:
            self._mode = _Mode.IDLE

    def record(self):
        return self._enter(_Mode.RECORD)

    def replay(self):
        return self._enter(_Mode.REPLAY)

    def record_invocation(self, task: UnitTask, task_input: TaskInput, task_output: TaskOutput) -> None:
        if not self.is_recording:
            raise RuntimeError("Task invocation can only be recorded in recording mode.")
        self.invocations.append(TaskInvocation(task=task.model_copy(deep=True),
                                               task_input=task_input.model_copy(deep=True),
                                               task_output=task_output.model_copy(deep=True)))

    async def dispatch_tasks_and_wait(self) -> None:
        if self._mode is not _Mode.IDLE:
            raise RuntimeError("Cannot dispatch tasks while recording or replaying.")
        if not self.invocations:
            logger.warning("No task invocations were recorded. Finishing dispatch immediately.")
            return
        if self.task_outputs:
            raise RuntimeError("Task outputs already exist. Task contexts are not supposed to be reused.")
        with tracer.start_as_current_span("TaskContext.dispatch_tasks_and_wait") as span:
            graph = TaskGraphDispatch(invocations=self.invocations)
            manager = task_manager_context.get()
            if manager is None:
                url = os.environ.get("CORNSERVE_GATEWAY_URL", GATEWAY_URL) + "/tasks/invoke"
                outputs = await graph.dispatch(url, client=get_client())
            else:
                try:
                    outputs = await manager.invoke_tasks(graph)
                except Exception as e:
                    logger.exception("Failed to invoke tasks: %s", e)
                    raise RuntimeError("Failed to invoke tasks.") from e
            for i, (inv, out) in enumerate(zip(self.invocations, outputs, strict=True)):
                parsed = type(inv.task_output).model_validate(out)
                span.set_attribute(f"task_context.task.{i}.output", parsed.model_dump_json())
                self.task_outputs[inv.task.id].append(parsed)

    def replay_invocation(self, task: Task) -> TaskOutput:
        """Outputs of one task id are handed out in the order its invocations were recorded."""
        if not self.is_replaying:
            raise RuntimeError("Task context is not in replay mode.")
        if not self.task_outputs:
            raise RuntimeError("No task outputs exist.")
        if task.id not in self.task_outputs:
            raise RuntimeError(f"Task {task.id} not found in task outputs.")
        try:
            return self.task_outputs[task.id].popleft()
        except IndexError as e:
            raise RuntimeError(f"Task {task.id} has no more outputs to replay.") from e


class UnitTaskList(BaseModel):
    """Serialisable list of unit tasks: ``{"_task_list": [{"class_name", "task": <json>}]}``."""

    tasks: list[UnitTask]

    model_config = ConfigDict(arbitrary_types_allowed=True)

    @model_serializer()
    def _dump(self) -> dict[str, Any]:
        return {"_task_list": [{"class_name": type(t).__name__, "task": t.model_dump_json()} for t in self.tasks]}

    @model_validator(mode="before")
    @classmethod
    def _load(cls, data: Any):
        if not isinstance(data, dict) or "_task_list" not in data:
            return data
        tasks = []
        for item in data["_task_list"]:
            task_cls, _, _ = _unit_task_classes(item["class_name"])
            tasks.append(task_cls.model_validate_json(item["task"]))
        return {"tasks": tasks}
