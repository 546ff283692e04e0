"""llm.c tokenizer files and sampling (reference: example/common/tokenizer.cc:39-146).

File: 1024-byte header (uint32 magic 20240328 GPT-2 / 20240801 LLaMA-3, uint32 version 1|2,
uint32 vocab_size, [uint32 eot when version 2]) then ``vocab_size`` entries of ``{uint8 len, bytes}``.
Sampling: xorshift* generator seeded with 1337, multinomial over the softmax of position ``t - 1``,
prompt "The meaning of life is".
"""
from __future__ import annotations

import struct
from typing import List, Optional

import torch

kGpt2Magic, kLlama3Magic = 20240328, 20240801
kGpt2Eot, kLlama3Eot = 50256, 128001
kPromptMap = {kGpt2Magic: [464, 3616, 286, 1204, 318], kLlama3Magic: [791, 7438, 315, 2324, 374]}
_MASK64 = (1 << 64) - 1


def RandomU32(state: List[int]) -> int:
    """xorshift*: ``state`` is a one-element list holding the 64-bit state."""
    s = state[0]
    s ^= s >> 12
    s ^= (s << 25) & _MASK64
    s ^= s >> 27
    state[0] = s
    return ((s * 0x2545F4914F6CDD1D) & _MASK64) >> 32


def RandomF32(state: List[int]) -> float:
    return (RandomU32(state) >> 8) / 16777216.0


def SampleMult(probabilities, coin: float) -> int:
    cdf = torch.cumsum(probabilities.float(), 0)
    idx = int(torch.searchsorted(cdf, torch.tensor(coin), right=True).item())
    return min(idx, probabilities.numel() - 1)


def write_tokenizer_file(path: str, tokens: List[bytes], magic: int = kGpt2Magic, version: int = 2, eot: int = 0):
    header = bytearray(1024)
    struct.pack_into("<III", header, 0, magic, version, len(tokens))
    if version == 2:
        struct.pack_into("<I", header, 12, eot)
    with open(path, "wb") as f:
        f.write(header)
        for t in tokens:
            f.write(struct.pack("<B", len(t)))
            f.write(t)


class Tokenizer:
    def __init__(self, filepath: str):
        with open(filepath, "rb") as f:
            header = f.read(1024)
            self.magic_number, version, self.vocab_size = struct.unpack_from("<III", header, 0)
            if self.magic_number not in kPromptMap:
                raise ValueError(f"Unsupported tokenizer magic: {self.magic_number}")
            if version == 1:
                self.eot_token = kGpt2Eot if self.magic_number == kGpt2Magic else kLlama3Eot
            elif version == 2:
                (self.eot_token,) = struct.unpack_from("<I", header, 12)
            else:
                raise ValueError(f"Unsupported tokenizer version: {version}")
            self.token_table: List[bytes] = []
            for _ in range(self.vocab_size):
                (n,) = struct.unpack("<B", f.read(1))
                self.token_table.append(f.read(n))

    def Decode(self, token_id: int) -> str:
        if token_id >= self.vocab_size:
            return "[INVALID_TOKEN]"
        return self.token_table[token_id].decode("utf-8", errors="replace")

    def GetEndOfText(self) -> int:
        return self.eot_token

    def GenerateText(self, model, batch_size: int, sequence_length: int, text_length: int, device,
                     print_fn=print) -> str:
        """Greedy-free sampling loop of the reference: the whole ``[B, T]`` window is re-run for
        every new token and position ``t - 1`` of row 0 is sampled."""
        x = torch.full((batch_size, sequence_length), self.eot_token, dtype=torch.int64)
        prompt = kPromptMap[self.magic_number]
        x.view(-1)[: len(prompt)] = torch.tensor(prompt)
        state = [1337]
        out = ["The meaning of life is"]
        dev = device.torch_device() if hasattr(device, "torch_device") else torch.device(device)
        with torch.no_grad():
            for t in range(len(prompt), text_length):
                logits = model(x.to(dev))
                probs = torch.softmax(logits[0, t - 1].float(), -1).cpu()
                nxt = SampleMult(probs, RandomF32(state))
                x.view(-1)[t] = nxt
                out.append(self.Decode(nxt))
        text = "".join(out)
        if print_fn:
            print_fn(text)
        return text
