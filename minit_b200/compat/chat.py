"""The interfaces the reference's example servers subclass (minit/chat/server.py:12-34, sample.py:5-14,
template.py:5-20, tokenizer.py:5-48, agent.py:10-59): a ``Server`` decodes token ids into next-token scores for a
session, a ``Tokenizer`` maps text to ids and back, a ``Template`` wraps the chat turns, a ``Sampler`` picks a token,
and an ``Agent`` session loops them until the template's end marker.  Only what the example scripts name is here; the
scripts bring their own models."""
from __future__ import annotations

from typing import Callable, Generic, List, Optional, Tuple, TypeVar

_Session = TypeVar("_Session")


class Server(Generic[_Session]):
    def decode(self, session: _Session, input_ids: List[int]):
        raise NotImplementedError()

    def create_session(self) -> _Session:
        raise NotImplementedError()


class CacheInputSession:
    """a session that re-sends the whole conversation every step"""

    def __init__(self, input_ids: Optional[List[int]] = None) -> None:
        self.input_ids: List[int] = [] if input_ids is None else input_ids


class CacheKeyValueSession:
    """a session that keeps the per-layer (key, value) caches and the number of tokens they hold"""

    def __init__(self, kv_cache_list: List[Tuple[object, object]]) -> None:
        self.kv_cache_list = kv_cache_list
        self.offset = 0


class Sampler:
    def sample(self, probs) -> int:
        raise NotImplementedError()


class Top1Sampler(Sampler):
    def sample(self, probs) -> int:
        return int(probs.numpy().argmax(axis=-1).item())


class Template:
    def generate_header(self) -> str:
        raise NotImplementedError()

    def generate_prompt(self, prompt: str) -> str:
        raise NotImplementedError()

    def generate(self, user: str) -> Tuple[str, str]:
        raise NotImplementedError()

    def eos(self) -> str:
        raise NotImplementedError()


class Tokenizer:
    def tokenize(self, text: str) -> List[int]:
        raise NotImplementedError()

    def detokenize(self, ids: List[int]) -> str:
        raise NotImplementedError()


class SentencePieceTokenizer(Tokenizer):
    def __init__(self, path: str) -> None:
        import sentencepiece
        self.sentence_piece = sentencepiece.SentencePieceProcessor(path)

    def tokenize(self, text: str) -> List[int]:
        (input_ids,) = self.sentence_piece.tokenize([text])
        return input_ids

    def detokenize(self, ids: List[int]) -> str:
        return "".join(self.sentence_piece.id_to_piece(i) for i in ids)


class HuggingFaceTokenizer(Tokenizer):
    def __init__(self, path: str) -> None:
        import transformers
        self.hugging_face = transformers.PreTrainedTokenizerFast(tokenizer_file=path)

    def tokenize(self, text: str) -> List[int]:
        return self.hugging_face.encode(text, add_special_tokens=False)

    def detokenize(self, ids: List[int]) -> str:
        return "".join(self.hugging_face.decode(i) for i in ids)


class Agent:
    class Session:
        def __init__(self, server: Server, tokenizer: Tokenizer, template: Template, sampler: Sampler, prompt: Optional[str]) -> None:
            session = server.create_session()
            self.decoder: Callable[[List[int]], object] = lambda input_ids: server.decode(session, input_ids)
            self.tokenizer, self.template, self.sampler = tokenizer, template, sampler
            header = template.generate_header()
            if prompt is not None:
                header += template.generate_prompt(prompt)
            if header:
                self.decoder(tokenizer.tokenize(header))

        def interact(self, user: str) -> str:
            prefix, postfix = self.template.generate(user)
            eos = self.template.eos()
            reply = ""
            input_ids = self.tokenizer.tokenize(prefix)
            while True:
                output_id = self.sampler.sample(self.decoder(input_ids))
                piece = self.tokenizer.detokenize([output_id])
                if piece == eos:
                    break
                reply += piece
                input_ids = [output_id]
            self.decoder(self.tokenizer.tokenize(postfix))
            return reply

    def __init__(self, server: Server, tokenizer: Tokenizer, template: Template, sampler: Sampler) -> None:
        self.server, self.tokenizer, self.template, self.sampler = server, tokenizer, template, sampler

    def create_session(self, prompt: Optional[str]) -> "Agent.Session":
        return Agent.Session(self.server, self.tokenizer, self.template, self.sampler, prompt)


def chat_cmdline(agent: Agent, prompt: Optional[str]) -> None:
    """a read-answer loop on the terminal"""
    session = agent.create_session(prompt)
    while True:
        try:
            user = input("> ")
        except EOFError:
            return
        print(session.interact(user))
