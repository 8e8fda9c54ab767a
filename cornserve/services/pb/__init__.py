"""Protocol-buffer messages and gRPC bindings of the five ``proto/v1`` files.

The schema lives in :data:`SCHEMA` (one entry per ``.proto`` file).  Message classes are built at import
time from ``FileDescriptorProto`` objects, so no code generator is needed at build time, and the
``proto/v1/*.proto`` files are emitted from the same table (``python -m cornserve.services.pb proto/v1``),
which keeps text and bindings in lock-step.  Package names, message names, field names and field
numbers are those of the reference RPC surface (proto/v1/*.proto), so either side can talk to the other.

Each file is exposed like generated code: ``sidecar_pb2.SendRequest``, ``sidecar_pb2_grpc.SidecarStub``,
``sidecar_pb2_grpc.SidecarServicer``, ``sidecar_pb2_grpc.add_SidecarServicer_to_server``.
"""

from __future__ import annotations

import types
from typing import Any

import grpc
from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

F = descriptor_pb2.FieldDescriptorProto

_SCALARS = {
    "string": F.TYPE_STRING, "int32": F.TYPE_INT32, "int64": F.TYPE_INT64, "bool": F.TYPE_BOOL,
    "bytes": F.TYPE_BYTES, "float": F.TYPE_FLOAT, "double": F.TYPE_DOUBLE, "uint32": F.TYPE_UINT32,
}

# field = (name, number, type[, label])   type: scalar | "Msg" | "pkg.Msg" | "enum:Name" | "map<string,Msg>"
# label: "" | "repeated" | "optional"
STATUS = ("status", 1, "enum:common.Status")
SCHEMA: dict[str, dict[str, Any]] = {
    "common": {
        "package": "cornserve.common", "imports": [],
        "enums": {"Status": [("STATUS_UNSPECIFIED", 0), ("STATUS_OK", 1), ("STATUS_ERROR", 2)]},
        "messages": {
            "SyncTaskRegistryRequest": [],
            "SyncTaskRegistryResponse": [STATUS],
        },
        "services": {},
    },
    "resource_manager": {
        "package": "cornserve.resource_manager", "imports": ["common"], "enums": {},
        "messages": {
            "DeployUnitTaskRequest": [("task_instance_name", 1, "string")],
            "DeployUnitTaskResponse": [STATUS],
            "TeardownUnitTaskRequest": [("task_instance_name", 1, "string")],
            "TeardownUnitTaskResponse": [STATUS],
            "TaskManagerStatus": [("task_instance_name", 1, "string"), ("status", 2, "enum:common.Status")],
            "HealthcheckRequest": [],
            "HealthcheckResponse": [STATUS, ("task_manager_statuses", 2, "TaskManagerStatus", "repeated")],
            "ScaleUnitTaskRequest": [("task_instance_name", 1, "string"), ("num_gpus", 2, "int32")],
            "ScaleUnitTaskResponse": [STATUS],
        },
        "services": {"ResourceManager": [
            ("DeployUnitTask", "DeployUnitTaskRequest", "DeployUnitTaskResponse"),
            ("TeardownUnitTask", "TeardownUnitTaskRequest", "TeardownUnitTaskResponse"),
            ("Healthcheck", "HealthcheckRequest", "HealthcheckResponse"),
            ("ScaleUnitTask", "ScaleUnitTaskRequest", "ScaleUnitTaskResponse"),
            ("SyncTaskRegistry", "common.SyncTaskRegistryRequest", "common.SyncTaskRegistryResponse"),
        ]},
    },
    "task_manager": {
        "package": "cornserve.task_manager", "imports": ["common"],
        "enums": {"ResourceAction": [("ADD", 0), ("REMOVE", 1)]},
        "messages": {
            "GPUResource": [("action", 1, "enum:ResourceAction"), ("node_id", 2, "string"), ("global_rank", 3, "int32"),
                            ("local_rank", 4, "int32")],
            "RegisterTaskRequest": [("task_manager_id", 1, "string"), ("task_instance_name", 2, "string"),
                                    ("gpus", 3, "GPUResource", "repeated")],
            "RegisterTaskResponse": [STATUS],
            "UpdateResourcesRequest": [("task_manager_id", 1, "string"), ("gpus", 2, "GPUResource", "repeated")],
            "UpdateResourcesResponse": [STATUS],
            "ShutdownRequest": [],
            "ShutdownResponse": [STATUS],
            "ReconcileTargetLoadRequest": [("task_id", 1, "string"), ("target_load", 2, "float")],
            "ReconcileTargetLoadResponse": [STATUS, ("message", 2, "string")],
            "DeploymentConfig": [("num_replicas", 1, "int32"), ("tensor_parallel_degree", 2, "int32"),
                                 ("pipeline_parallel_degree", 3, "int32"), ("gpu_assignments", 4, "string", "repeated")],
            "ProfilePoint": [("num_gpus", 1, "int32"), ("max_sustainable_load", 2, "float"),
                             ("deployment_config", 3, "DeploymentConfig")],
            "GetTaskProfileRequest": [("task_id", 1, "string")],
            "GetTaskProfileResponse": [("profile_points", 1, "ProfilePoint", "repeated")],
            "GetRouteRequest": [("request_id", 1, "string"), ("routing_hint", 2, "string", "optional")],
            "GetRouteResponse": [("task_executor_url", 1, "string"), ("sidecar_ranks", 2, "int32", "repeated")],
            "TaskExecutorStatus": [STATUS, ("sidecar_ranks", 2, "int32", "repeated")],
            "HealthcheckRequest": [],
            "HealthcheckResponse": [STATUS, ("task_executor_statuses", 2, "map<string,TaskExecutorStatus>")],
        },
        "services": {"TaskManager": [
            ("RegisterTask", "RegisterTaskRequest", "RegisterTaskResponse"),
            ("UpdateResources", "UpdateResourcesRequest", "UpdateResourcesResponse"),
            ("Shutdown", "ShutdownRequest", "ShutdownResponse"),
            ("GetTaskProfile", "GetTaskProfileRequest", "GetTaskProfileResponse"),
            ("ReconcileTargetLoad", "ReconcileTargetLoadRequest", "ReconcileTargetLoadResponse"),
            ("GetRoute", "GetRouteRequest", "GetRouteResponse"),
            ("Healthcheck", "HealthcheckRequest", "HealthcheckResponse"),
            ("SyncTaskRegistry", "common.SyncTaskRegistryRequest", "common.SyncTaskRegistryResponse"),
        ]},
    },
    "task_dispatcher": {
        "package": "cornserve.task_dispatcher", "imports": ["common"], "enums": {},
        "messages": {
            "TaskManagerDeployment": [("url", 1, "string")],
            "NotifyUnitTaskDeploymentRequest": [("task_instance_name", 1, "string"),
                                                ("task_manager", 2, "TaskManagerDeployment")],
            "NotifyUnitTaskDeploymentResponse": [STATUS],
            "NotifyUnitTaskTeardownRequest": [("task_instance_name", 1, "string")],
            "NotifyUnitTaskTeardownResponse": [STATUS],
        },
        "services": {"TaskDispatcher": [
            ("NotifyUnitTaskDeployment", "NotifyUnitTaskDeploymentRequest", "NotifyUnitTaskDeploymentResponse"),
            ("NotifyUnitTaskTeardown", "NotifyUnitTaskTeardownRequest", "NotifyUnitTaskTeardownResponse"),
            ("SyncTaskRegistry", "common.SyncTaskRegistryRequest", "common.SyncTaskRegistryResponse"),
        ]},
    },
    "sidecar": {
        "package": "cornserve.sidecar", "imports": ["common"],
        "enums": {"HealthStatus": [("HEALTH_ALL_GOOD", 0), ("HEALTH_MEMORY_PRESSURE", 1), ("HEALTH_OFFLINE", 2)]},
        "messages": {
            "RegisterRequest": [("rank", 1, "int32"), ("group", 2, "int32", "repeated"), ("send_slot_numel", 3, "int32"),
                                ("recv_slot_numel", 4, "int32"), ("concurrent_copy", 5, "bool"),
                                ("send_dtype", 6, "string"), ("recv_dtype", 7, "string")],
            "RegisterResponse": [STATUS, ("shm_size", 2, "int64"), ("local_rank", 3, "int32"),
                                 ("num_local_sidecars", 4, "int32")],
            "RankGroup": [("ranks", 1, "int32", "repeated")],
            "CloseStreamRequest": [("id", 1, "string"), ("num_chunks", 2, "int32")],
            "CloseStreamResponse": [STATUS],
            "SendRequest": [("id", 1, "string"), ("dst_ranks", 2, "RankGroup", "repeated"), ("shard_rank", 3, "int32"),
                            ("data", 4, "bytes"), ("chunk_id", 5, "int32"), ("num_chunks", 6, "int32")],
            "SendResponse": [STATUS],
            "ReceiveRequest": [("id", 1, "string"), ("chunk_id", 2, "int32")],
            "ReceiveResponse": [STATUS, ("data", 2, "bytes")],
            "MarkDoneRequest": [("id", 1, "string"), ("chunk_id", 2, "int32"), ("shard_rank", 3, "int32")],
            "MarkDoneResponse": [STATUS],
            "UnlinkRequest": [("id", 1, "string"), ("chunk_id", 2, "int32")],
            "UnlinkResponse": [STATUS],
            "PrepareReceiveRequest": [("id", 1, "string"), ("data", 2, "bytes"), ("src_rank", 3, "int32"),
                                      ("chunk_id", 4, "int32"), ("num_chunks", 5, "int32")],
            "PrepareReceiveResponse": [STATUS],
            "CheckHealthRequest": [],
            "CheckHealthResponse": [("status", 1, "enum:HealthStatus")],
            "ReportMemoryRequest": [("pressure", 1, "int32")],
            "ReportMemoryResponse": [STATUS],
        },
        "services": {"Sidecar": [
            ("Register", "RegisterRequest", "RegisterResponse"),
            ("Send", "SendRequest", "SendResponse"),
            ("Receive", "ReceiveRequest", "ReceiveResponse"),
            ("MarkDone", "MarkDoneRequest", "MarkDoneResponse"),
            ("Unlink", "UnlinkRequest", "UnlinkResponse"),
            ("PrepareReceive", "PrepareReceiveRequest", "PrepareReceiveResponse"),
            ("CheckHealth", "CheckHealthRequest", "CheckHealthResponse"),
            ("CloseStream", "CloseStreamRequest", "CloseStreamResponse"),
        ]},
    },
}

_ORDER = ["common", "resource_manager", "task_manager", "task_dispatcher", "sidecar"]
_pool = descriptor_pool.DescriptorPool()


def _qualify(name: str, file_key: str) -> str:
    """``Msg`` -> ``.cornserve.<file>.Msg``; ``common.Msg`` -> ``.cornserve.common.Msg``."""
    if "." in name:
        f, n = name.split(".", 1)
        return f".{SCHEMA[f]['package']}.{n}"
    return f".{SCHEMA[file_key]['package']}.{name}"


def _camel(s: str) -> str:
    return "".join(p.capitalize() for p in s.split("_"))


def _build_file(key: str) -> descriptor_pb2.FileDescriptorProto:
    spec = SCHEMA[key]
    fd = descriptor_pb2.FileDescriptorProto(name=f"{key}.proto", package=spec["package"], syntax="proto3")
    fd.dependency.extend(f"{d}.proto" for d in spec["imports"])
    for ename, values in spec["enums"].items():
        e = fd.enum_type.add(name=ename)
        for vname, num in values:
            e.value.add(name=vname, number=num)
    for mname, fields in spec["messages"].items():
        m = fd.message_type.add(name=mname)
        for field in fields:
            fname, num, ftype = field[:3]
            label = field[3] if len(field) > 3 else ""
            f = m.field.add(name=fname, number=num, json_name=fname)
            f.label = F.LABEL_REPEATED if label == "repeated" else F.LABEL_OPTIONAL
            if ftype.startswith("map<"):
                ktype, vtype = ftype[4:-1].split(",")
                entry = m.nested_type.add(name=_camel(fname) + "Entry")
                entry.options.map_entry = True
                entry.field.add(name="key", number=1, label=F.LABEL_OPTIONAL, type=_SCALARS[ktype.strip()])
                v = entry.field.add(name="value", number=2, label=F.LABEL_OPTIONAL, type=F.TYPE_MESSAGE)
                v.type_name = _qualify(vtype.strip(), key)
                f.label = F.LABEL_REPEATED
                f.type = F.TYPE_MESSAGE
                f.type_name = f".{spec['package']}.{mname}.{entry.name}"
            elif ftype in _SCALARS:
                f.type = _SCALARS[ftype]
            elif ftype.startswith("enum:"):
                f.type = F.TYPE_ENUM
                f.type_name = _qualify(ftype[5:], key)
            else:
                f.type = F.TYPE_MESSAGE
                f.type_name = _qualify(ftype, key)
            if label == "optional":
                f.proto3_optional = True
                oneof_index = len(m.oneof_decl)
                m.oneof_decl.add(name=f"_{fname}")
                f.oneof_index = oneof_index
    for sname, methods in spec["services"].items():
        s = fd.service.add(name=sname)
        for mname, req, resp in methods:
            s.method.add(name=mname, input_type=_qualify(req, key), output_type=_qualify(resp, key))
    return fd


def _message_class(full_name: str):
    return message_factory.GetMessageClass(_pool.FindMessageTypeByName(full_name))


def _make_modules(key: str) -> tuple[types.ModuleType, types.ModuleType]:
    spec = SCHEMA[key]
    pb2 = types.ModuleType(f"{__name__}.{key}_pb2")
    pb2.DESCRIPTOR = _pool.FindFileByName(f"{key}.proto")
    for mname in spec["messages"]:
        setattr(pb2, mname, _message_class(f"{spec['package']}.{mname}"))
    for ename, values in spec["enums"].items():
        ed = _pool.FindEnumTypeByName(f"{spec['package']}.{ename}")
        ns = types.SimpleNamespace(**{v: n for v, n in values})
        ns.Name = lambda n, ed=ed: ed.values_by_number[n].name
        ns.Value = lambda s, ed=ed: ed.values_by_name[s].number
        ns.DESCRIPTOR = ed
        setattr(pb2, ename, ns)
        for v, n in values:
            setattr(pb2, v, n)  # generated code also exports enum values at module level

    rpc = types.ModuleType(f"{__name__}.{key}_pb2_grpc")
    for sname, methods in spec["services"].items():
        full = f"{spec['package']}.{sname}"
        resolved = [(m, _message_class(_qualify(req, key)[1:]), _message_class(_qualify(resp, key)[1:]))
                    for m, req, resp in methods]

        def stub_init(self, channel, _methods=resolved, _full=full):
            for m, req, resp in _methods:
                setattr(self, m, channel.unary_unary(f"/{_full}/{m}", request_serializer=req.SerializeToString,
                                                     response_deserializer=resp.FromString))

        stub = type(f"{sname}Stub", (), {"__init__": stub_init, "__doc__": f"Client stub of {full}."})

        def _unimplemented(name):
            def method(self, request, context):
                context.set_code(grpc.StatusCode.UNIMPLEMENTED)
                context.set_details(f"{name} is not implemented")
                raise NotImplementedError(f"{name} is not implemented")
            return method

        servicer = type(f"{sname}Servicer", (), {m: _unimplemented(m) for m, _, _ in resolved})

        def add_to_server(servicer_obj, server, _methods=resolved, _full=full):
            handlers = {
                m: grpc.unary_unary_rpc_method_handler(getattr(servicer_obj, m), request_deserializer=req.FromString,
                                                       response_serializer=resp.SerializeToString)
                for m, req, resp in _methods
            }
            server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(_full, handlers),))

        setattr(rpc, f"{sname}Stub", stub)
        setattr(rpc, f"{sname}Servicer", servicer)
        setattr(rpc, f"add_{sname}Servicer_to_server", add_to_server)
    return pb2, rpc


for _key in _ORDER:
    _pool.Add(_build_file(_key))

common_pb2, _ = _make_modules("common")
resource_manager_pb2, resource_manager_pb2_grpc = _make_modules("resource_manager")
task_manager_pb2, task_manager_pb2_grpc = _make_modules("task_manager")
task_dispatcher_pb2, task_dispatcher_pb2_grpc = _make_modules("task_dispatcher")
sidecar_pb2, sidecar_pb2_grpc = _make_modules("sidecar")


def emit_proto(key: str) -> str:
    """Text of ``proto/v1/<key>.proto`` generated from :data:`SCHEMA`."""
    spec = SCHEMA[key]
    out = ['syntax = "proto3";', "", f"package {spec['package']};", ""]
    for imp in spec["imports"]:
        out.append(f'import "{imp}.proto";')
    if spec["imports"]:
        out.append("")
    for sname, methods in spec["services"].items():
        out.append(f"service {sname} {{")
        for m, req, resp in methods:
            out.append(f"  rpc {m}({req}) returns ({resp});")
        out += ["}", ""]
    for ename, values in spec["enums"].items():
        out.append(f"enum {ename} {{")
        out += [f"  {v} = {n};" for v, n in values]
        out += ["}", ""]
    for mname, fields in spec["messages"].items():
        if not fields:
            out += [f"message {mname} {{}}", ""]
            continue
        out.append(f"message {mname} {{")
        for field in fields:
            fname, num, ftype = field[:3]
            label = field[3] if len(field) > 3 else ""
            t = ftype[5:] if ftype.startswith("enum:") else ftype.replace("<string,", "<string, ")
            out.append(f"  {label + ' ' if label else ''}{t} {fname} = {num};")
        out += ["}", ""]
    return "\n".join(out)


def write_proto_files(dest) -> list[str]:
    import pathlib

    dest = pathlib.Path(dest)
    dest.mkdir(parents=True, exist_ok=True)
    written = []
    for k in _ORDER:
        (dest / f"{k}.proto").write_text(emit_proto(k))
        written.append(str(dest / f"{k}.proto"))
    return written
