"""`/v1/embeddings`, `/v1/rerank`, `/v1/score` (reference `entrypoints/openai/serving_{embedding,rerank,score}.py`)."""

from __future__ import annotations

from ...managers.io_struct import EmbeddingReqInput
from .protocol import (EmbeddingObject, EmbeddingRequest, EmbeddingResponse, RerankResponse, ScoringRequest,
                       ScoringResponse, UsageInfo, V1RerankReqInput)
from .serving_base import OpenAIServingBase


class OpenAIServingEmbedding(OpenAIServingBase):
    def _validate_request(self, request: EmbeddingRequest):
        if isinstance(request.input, (str, list)) and len(request.input) == 0:
            return "Input cannot be empty"
        return None

    def _convert_to_internal_request(self, request: EmbeddingRequest):
        inp = request.input
        if isinstance(inp, str) or (isinstance(inp, list) and inp and isinstance(inp[0], str)):
            return EmbeddingReqInput(text=inp, rid=request.rid), request
        return EmbeddingReqInput(input_ids=inp, rid=request.rid), request

    async def _handle_non_streaming_request(self, adapted, request, raw_request):
        ret = await self.tokenizer_manager.generate_request(adapted, raw_request).__anext__()
        if not isinstance(ret, list):
            ret = [ret]
        data = [EmbeddingObject(embedding=r["embedding"], index=i) for i, r in enumerate(ret)]
        pt = sum(r["meta_info"]["prompt_tokens"] for r in ret)
        return EmbeddingResponse(data=data, model=request.model, usage=UsageInfo(prompt_tokens=pt, total_tokens=pt))


class OpenAIServingRerank(OpenAIServingBase):
    def _convert_to_internal_request(self, request: V1RerankReqInput):
        pairs = [f"{request.query}</s>{d}" for d in request.documents]
        return EmbeddingReqInput(text=pairs), request

    async def _handle_non_streaming_request(self, adapted, request, raw_request):
        ret = await self.tokenizer_manager.generate_request(adapted, raw_request).__anext__()
        out = [RerankResponse(score=float(r["embedding"][0]), document=d, index=i, meta_info=r["meta_info"])
               for i, (r, d) in enumerate(zip(ret, request.documents))]
        return sorted(out, key=lambda x: -x.score)


class OpenAIServingScore(OpenAIServingBase):
    def _convert_to_internal_request(self, request: ScoringRequest):
        return request, request

    async def _handle_non_streaming_request(self, adapted, request, raw_request):
        scores = await self.tokenizer_manager.score_request(
            query=request.query, items=request.items, label_token_ids=request.label_token_ids,
            apply_softmax=request.apply_softmax, item_first=request.item_first, request=raw_request)
        return ScoringResponse(scores=scores, model=request.model)
