"""Task programming model: root-class inference, (de)serialisation, equivalence, streams, sub-task
registration, record mode of the composite tasks (no services needed)."""

import asyncio
import json

import pytest

from cornserve.task.base import (Stream, Task, TaskContext, TaskGraphDispatch, TaskInvocation, TaskOutput,
                                      UnitTaskList, discover_unit_tasks, task_context)
from cornserve.task.forward import DataForward, ForwardableType, Tensor
from cornserve_tasklib import (DisaggregatedMLLMTask, EncoderInput, EncoderTask, LLMEmbeddingUnitTask, LLMUnitTask,
                                    MLLMEmbeddingTask, MLLMTask, Modality, OmniInput, OmniTask,
                                    OpenAIChatCompletionChunk, OpenAIChatCompletionRequest)
from cornserve_tasklib.task.unit.generator import AudioGeneratorTask

MODEL = "Qwen/Qwen2.5-VL-7B-Instruct"


def _request(n_images=2, n_audio=0, model=MODEL):
    content = [{"type": "text", "text": "describe"}]
    content += [{"type": "image_url", "image_url": {"url": f"http://x/{i}.png"}} for i in range(n_images)]
    content += [{"type": "audio_url", "audio_url": {"url": f"http://x/{i}.wav"}} for i in range(n_audio)]
    return OpenAIChatCompletionRequest(model=model, messages=[{"role": "user", "content": content}])


def test_root_unit_task_cls():
    assert EncoderTask.root_unit_task_cls is EncoderTask
    assert LLMUnitTask.root_unit_task_cls.__name__ == "LLMBaseUnitTask"
    assert LLMEmbeddingUnitTask.root_unit_task_cls is LLMUnitTask.root_unit_task_cls

    class Sub(EncoderTask):
        note: str = ""

    assert Sub.root_unit_task_cls is EncoderTask


def test_invoke_must_be_sync():
    with pytest.raises(TypeError):
        class Bad(Task[EncoderInput, TaskOutput]):  # noqa: F841
            async def invoke(self, task_input):
                return TaskOutput()


def test_data_forward_types():
    assert DataForward[Tensor]().data_type == ForwardableType.TENSOR
    assert DataForward[dict]().data_type == ForwardableType.DICT
    with pytest.raises(ValueError):
        DataForward()


def test_invocation_serde_roundtrip():
    enc = EncoderTask(modality=Modality.IMAGE, model_ids={MODEL})
    inp = EncoderInput(model_id=MODEL, data_urls=["a", "b"])
    inv = TaskInvocation(task=enc, task_input=inp, task_output=enc.make_record_output(inp))
    wire = json.loads(json.dumps(inv.model_dump()))
    assert wire["class_name"] == "EncoderTask" and set(wire["body"]) == {"task", "task_input", "task_output"}
    back = TaskInvocation.model_validate(wire)
    assert back.task.id == enc.id and back.task_input == inp
    assert [f.id for f in back.task_output.embeddings] == [f.id for f in inv.task_output.embeddings]
    lst = UnitTaskList.model_validate(json.loads(json.dumps(UnitTaskList(tasks=[enc]).model_dump())))
    assert lst.tasks[0].is_equivalent_to(enc)


def test_equivalence():
    a = EncoderTask(modality=Modality.IMAGE, model_ids={MODEL})
    b = EncoderTask(modality=Modality.IMAGE, model_ids={MODEL})
    c = EncoderTask(modality=Modality.VIDEO, model_ids={MODEL})
    assert a.id != b.id and a.is_equivalent_to(b) and not a.is_equivalent_to(c)
    assert LLMUnitTask(model_id=MODEL).is_equivalent_to(LLMEmbeddingUnitTask(model_id=MODEL))
    assert not LLMUnitTask(model_id=MODEL).is_equivalent_to(LLMUnitTask(model_id=MODEL, receive_embeddings=False))
    assert not a.is_equivalent_to("x")


def test_subtask_registration_and_discovery():
    t = MLLMTask(model_id=MODEL, modalities=[Modality.IMAGE, Modality.VIDEO])
    units = discover_unit_tasks([t])
    assert [type(u).__name__ for u in units] == ["EncoderTask", "EncoderTask", "LLMUnitTask"]
    assert len(t.subtask_attr_names) == 3
    o = OmniTask(modalities=[Modality.AUDIO])
    names = [type(u).__name__ for u in discover_unit_tasks([o])]
    assert names.count("EncoderTask") == 2 and "AudioGeneratorTask" in names and "OmniTalkerEmbeddingTask" in names


async def _lines(items):
    for i in items:
        yield i


def _chunk(text):
    return OpenAIChatCompletionChunk(id="1", choices=[{"index": 0, "delta": {"content": text}}]).model_dump_json()


def test_stream_iteration_and_transform():
    async def run():
        s = Stream[OpenAIChatCompletionChunk](async_iterator=_lines([_chunk("a"), "", _chunk("b")]))
        got = [c.choices[0].delta.content async for c in s]
        assert got == ["a", "b"]

        class Text(TaskOutput):
            text: str

        def to_text(c: OpenAIChatCompletionChunk) -> Text:
            return Text(text=c.choices[0].delta.content.upper())

        s = Stream[OpenAIChatCompletionChunk](async_iterator=_lines([_chunk("x"), _chunk("y")]))
        t = s.transform(to_text)
        assert s.async_iterator is None and t.item_type is Text
        assert [i.text async for i in t] == ["X", "Y"]
        with pytest.raises(ValueError):
            t.transform(to_text)
        with pytest.raises(ValueError):
            Stream[OpenAIChatCompletionChunk](async_iterator=_lines([])).transform(lambda c: c)
        raw = Stream[OpenAIChatCompletionChunk](async_iterator=_lines(["l1", " ", "l2"]))
        assert [r async for r in raw.aiter_raw()] == ["l1", "l2"]

    asyncio.run(run())


def _record(task, inp):
    ctx = TaskContext()
    task_context.set(ctx)
    with ctx.record():
        task.invoke(inp)
    return ctx.invocations


def test_mllm_record_per_url_and_coalesced():
    t = MLLMTask(model_id=MODEL, modalities=[Modality.IMAGE, Modality.AUDIO])
    invs = _record(t, _request(2, 1))
    assert [type(i.task).__name__ for i in invs] == ["EncoderTask"] * 3 + ["LLMUnitTask"]
    llm_in = invs[-1].task_input
    produced = [i.task_output.embeddings[0].id for i in invs[:3]]
    assert [f.id for f in llm_in.cornserve_embeddings] == produced
    assert TaskGraphDispatch(invocations=invs).is_streaming

    t = MLLMTask(model_id=MODEL, modalities=[Modality.IMAGE, Modality.AUDIO], coalesce_encoder_invocations=True)
    invs = _record(t, _request(2, 1))
    assert [type(i.task).__name__ for i in invs] == ["EncoderTask", "EncoderTask", "LLMUnitTask"]
    assert [len(i.task_input.data_urls) for i in invs[:2]] == [2, 1]
    order = [f.id for f in invs[-1].task_input.cornserve_embeddings]
    assert order == [f.id for f in invs[0].task_output.embeddings] + [invs[1].task_output.embeddings[0].id]

    with pytest.raises(ValueError):
        _record(MLLMTask(model_id=MODEL, modalities=[Modality.IMAGE]), _request(1, 1))
    no_fission = MLLMTask(model_id=MODEL, modalities=[Modality.IMAGE], encoder_fission=False)
    assert [type(i.task).__name__ for i in _record(no_fission, _request(2))] == ["LLMUnitTask"]


def test_concurrent_contexts_do_not_mix():
    t = MLLMTask(model_id=MODEL, modalities=[Modality.IMAGE])

    async def one(n):
        ctx = TaskContext()
        task_context.set(ctx)
        with ctx.record():
            await asyncio.sleep(0)
            t.invoke(_request(n))
        return len(ctx.invocations)

    async def run():
        return await asyncio.gather(*(asyncio.create_task(one(n)) for n in (1, 3, 2)))

    assert asyncio.run(run()) == [2, 4, 3]


def test_other_composites_record():
    invs = _record(MLLMEmbeddingTask(model_id=MODEL, modalities=[Modality.IMAGE]), _request(1))
    assert type(invs[-1].task).__name__ == "LLMEmbeddingUnitTask" and not TaskGraphDispatch(invocations=invs).is_streaming
    invs = _record(DisaggregatedMLLMTask(model_id=MODEL, modalities=[Modality.IMAGE]), _request(1))
    assert [type(i.task).__name__ for i in invs] == ["EncoderTask", "PrefillLLMUnitTask", "DecodeLLMUnitTask"]
    assert invs[2].task_input.cornserve_kv_transfer_params.id == invs[1].task_output.kv_transfer_params.id
    omni = OmniTask(modalities=[Modality.AUDIO])
    req = OmniInput(model=omni.model_id, messages=_request(0, 1, omni.model_id).messages)
    invs = _record(omni, req)
    assert [type(i.task).__name__ for i in invs] == ["EncoderTask", "LLMEmbeddingUnitTask", "OmniTalkerEmbeddingTask",
                                                      "AudioGeneratorTask"]
    assert invs[2].task_input.messages[-1].content == "<tts_pad>"
    assert invs[3].task_input.embeddings.id == invs[2].task_output.embeddings.id
    req.return_audio = False
    assert [type(i.task).__name__ for i in _record(omni, req)] == ["EncoderTask", "LLMUnitTask"]
    assert isinstance(AudioGeneratorTask(model_id="m").make_record_output(None), Stream)


def test_replay_returns_outputs_in_order():
    enc = EncoderTask(modality=Modality.IMAGE, model_ids={MODEL})
    ctx = TaskContext()
    task_context.set(ctx)
    inp = EncoderInput(model_id=MODEL, data_urls=["u"])
    with ctx.record():
        r1, r2 = enc.invoke(inp), enc.invoke(inp)
    ctx.task_outputs[enc.id].extend([r1, r2])
    with ctx.replay():
        assert enc.invoke(inp) is r1 and enc.invoke(inp) is r2
        with pytest.raises(RuntimeError):
            enc.invoke(inp)
    with pytest.raises(AssertionError):
        enc.invoke(inp)
