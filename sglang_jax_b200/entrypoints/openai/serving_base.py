"""Common request handling of the OpenAI endpoints (reference `entrypoints/openai/serving_base.py:24`):
validate -> convert to the engine's request type -> stream or not -> map errors to OpenAI errors."""

from __future__ import annotations

import json
import logging
from abc import ABC, abstractmethod
from typing import Any

from fastapi import Request
from fastapi.responses import ORJSONResponse, StreamingResponse

try:
    import orjson  # noqa: F401
    _JSON = ORJSONResponse
except Exception:  # orjson is optional
    from fastapi.responses import JSONResponse as _JSON

from .protocol import ErrorResponse

logger = logging.getLogger(__name__)


class OpenAIServingBase(ABC):
    def __init__(self, tokenizer_manager):
        self.tokenizer_manager = tokenizer_manager

    async def handle_request(self, request, raw_request: Request):
        try:
            err = self._validate_request(request)
            if err:
                return self.create_error_response(err)
            adapted, processed = self._convert_to_internal_request(request)
            if getattr(request, "stream", False):
                return await self._handle_streaming_request(adapted, processed, raw_request)
            return await self._handle_non_streaming_request(adapted, processed, raw_request)
        except ValueError as e:
            return self.create_error_response(str(e))
        except Exception as e:
            logger.exception("Error in request")
            return self.create_error_response(f"Internal server error: {e}", "InternalServerError", 500)

    def _validate_request(self, request) -> str | None:
        return None

    @abstractmethod
    def _convert_to_internal_request(self, request) -> tuple[Any, Any]: ...

    async def _handle_streaming_request(self, adapted, request, raw_request):
        return StreamingResponse(self._generate_stream(adapted, request, raw_request), media_type="text/event-stream")

    async def _generate_stream(self, adapted, request, raw_request):
        raise NotImplementedError
        yield  # pragma: no cover

    @abstractmethod
    async def _handle_non_streaming_request(self, adapted, request, raw_request): ...

    def create_error_response(self, message: str, err_type: str = "BadRequestError", status_code: int = 400,
                              param: str | None = None):
        err = ErrorResponse(message=message, type=err_type, param=param, code=status_code)
        return _JSON(content=err.model_dump(), status_code=status_code)

    def create_streaming_error_response(self, message: str, err_type: str = "BadRequestError",
                                        status_code: int = 400) -> str:
        err = ErrorResponse(message=message, type=err_type, code=status_code)
        return json.dumps({"error": err.model_dump()})
