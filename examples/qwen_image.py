"""Text-to-image with a user-defined composite task: the language model runs one step in embedding mode and forwards
its hidden states to the diffusion generator, which skips the system-prompt rows and returns a PNG.

    cornserve register examples/qwen_image.py
    cornserve invoke qwen_image '{"prompt": "A lighthouse at dawn", "height": 1024, "width": 1024, "num_inference_steps": 50}' \
        --png-key image --save-png-path lighthouse.png
"""

from __future__ import annotations

from cornserve.app.base import AppConfig
from cornserve.task.base import Task, TaskInput, TaskOutput
from cornserve_tasklib import ImageGeneratorInput, ImageGeneratorTask, LLMEmbeddingUnitTask, OpenAIChatCompletionRequest

TEXT_ENCODER = "Qwen/Qwen2.5-VL-7B-Instruct"
# the generator was trained with this instruction in front of every prompt; its 34 tokens are not part of the conditioning
SYSTEM_PROMPT = ("Describe the image by detailing the color, shape, size, texture, quantity, text, spatial relationships of "
                 "the objects and background:")
SYSTEM_PROMPT_TOKENS = 34


class ImageRequest(TaskInput):
    prompt: str
    height: int = 1024
    width: int = 1024
    num_inference_steps: int = 50


class ImageResponse(TaskOutput):
    image: str  # base64 PNG


class QwenImageTask(Task[ImageRequest, ImageResponse]):
    def post_init(self) -> None:
        self.text_encoder = LLMEmbeddingUnitTask(model_id=TEXT_ENCODER, receive_embeddings=False)
        self.generator = ImageGeneratorTask(model_id="Qwen/Qwen-Image")

    def invoke(self, task_input: ImageRequest) -> ImageResponse:
        chat = OpenAIChatCompletionRequest(model=TEXT_ENCODER, max_completion_tokens=1, messages=[
            {"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": task_input.prompt}])
        hidden = self.text_encoder.invoke(chat).embeddings
        out = self.generator.invoke(ImageGeneratorInput(height=task_input.height, width=task_input.width,
                                                        num_inference_steps=task_input.num_inference_steps,
                                                        skip_tokens=SYSTEM_PROMPT_TOKENS, embeddings=hidden))
        return ImageResponse(image=out.generated)


qwen_image = QwenImageTask()


class Config(AppConfig):
    tasks = {"qwen_image": qwen_image}


async def serve(request: ImageRequest) -> ImageResponse:
    return await qwen_image(request)
