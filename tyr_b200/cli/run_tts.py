"""Text-to-speech CLI (counterpart of Examples/Qwen3TTS/EndToEnd.lean and Examples/KittenTTSPretrained.lean).

    python -m tyr_b200.cli.run_tts qwen3tts --model-dir <dir> --text "Hello." --speaker vivian --wav-path out.wav
    python -m tyr_b200.cli.run_tts qwen3tts --model-dir <dir> --encode-audio-path ref.wav --encode-out-codes-path codes.txt --encode-only
    python -m tyr_b200.cli.run_tts qwen3tts --model-dir <dir> --text "Hi" --ref-audio-path ref.wav --streaming-decode --stream-chunk-frames 4
    python -m tyr_b200.cli.run_tts kitten <model_dir_or_repo> "<phonemes>" <voice> out.wav [speed]

Qwen3-TTS: text -> talker codes (``--codes-path``) -> waveform through the 12 Hz speech decoder (``--wav-path``); a reference
recording can be encoded to codec rows (``--encode-audio-path``) or turned into a speaker embedding (``--ref-audio-path``).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch


def parse_qwen(argv):
    p = argparse.ArgumentParser(prog="run_tts qwen3tts")
    p.add_argument("--model-dir", required=True)
    p.add_argument("--text", default="Hello from Tyr.")
    p.add_argument("--style-text", default=None, help="instruction text placed in front of the text (voice design models)")
    p.add_argument("--max-text-len", type=int, default=512)
    p.add_argument("--max-frames", type=int, default=256)
    p.add_argument("--language", default="auto")
    p.add_argument("--speaker", default=None)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--temperature", type=float, default=0.9)
    p.add_argument("--top-k", type=int, default=None)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--repetition-penalty", type=float, default=1.05)
    p.add_argument("--suppress-tail", type=int, default=1024)
    p.add_argument("--subtalker-temperature", type=float, default=0.9)
    p.add_argument("--subtalker-top-k", type=int, default=None)
    p.add_argument("--subtalker-top-p", type=float, default=1.0)
    p.add_argument("--subtalker-temp-by-group", default=None, help="comma-separated, one value per residual codebook")
    p.add_argument("--subtalker-top-k-by-group", default=None)
    p.add_argument("--subtalker-top-p-by-group", default=None)
    p.add_argument("--encode-audio-path", default=None)
    p.add_argument("--encode-out-codes-path", default="output/qwen3tts_ref_codes.txt")
    p.add_argument("--encode-only", action="store_true")
    p.add_argument("--codes-path", default="output/qwen3tts_codes.txt")
    p.add_argument("--wav-path", default="output/qwen3tts.wav")
    p.add_argument("--ref-audio-path", default=None, help="reference recording for voice cloning (base models)")
    p.add_argument("--speaker-mel-path", default="")
    p.add_argument("--speaker-mel-frames-path", default="")
    p.add_argument("--speech-tokenizer-dir", default=None)
    p.add_argument("--streaming-decode", action="store_true", help="decode audio while the talker is still generating")
    p.add_argument("--stream-chunk-frames", type=int, default=4)
    p.add_argument("--decode-chunk-size", type=int, default=300)
    p.add_argument("--decode-left-context", type=int, default=25)
    p.add_argument("--token-ids-path", default=None, help="whitespace-separated text token ids instead of --text")
    p.add_argument("--skip-decode", action="store_true")
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = p.parse_args(argv)
    if a.encode_only and not a.encode_audio_path:
        p.error("--encode-only requires --encode-audio-path")
    return a


def _floats(s):
    return None if s is None else [float(x) for x in s.split(",") if x.strip()]


def _ints(s):
    return None if s is None else [int(x) for x in s.split(",") if x.strip()]


def run_qwen(argv) -> int:
    from ..models import qwen3_tts as T
    from ..models import qwen3_tts_bridge as B
    from ..models import qwen3_tts_io as IO
    from ..io import media
    from ..tokenizer import hf as tok_hf
    a = parse_qwen(argv)
    model_dir = os.path.expanduser(a.model_dir)
    if a.encode_audio_path:
        rows, groups = B.encode_audio_to_codes(model_dir, a.encode_audio_path, a.encode_out_codes_path, a.device, a.speech_tokenizer_dir)
        print(f"encoded_codes={a.encode_out_codes_path} rows={rows} groups={groups}")
        if a.encode_only:
            return 0
    model = IO.load_sharded(model_dir, device=a.device, log=print)
    cfg = model.cfg
    if a.top_k is not None and a.top_k > cfg.talker.vocab_size:
        raise SystemExit(f"--top-k ({a.top_k}) exceeds talker vocab size ({cfg.talker.vocab_size})")
    if a.token_ids_path:
        ids = [int(t) for t in open(a.token_ids_path, encoding="utf-8").read().split()]
    else:
        ids = tok_hf.load_qwen3(model_dir).encode(a.text)
    ids = ids[:a.max_text_len]
    text_ids = torch.tensor([ids], dtype=torch.long)
    cond = {"language": a.language}
    if a.style_text:
        cond["instruct_ids"] = torch.tensor([tok_hf.load_qwen3(model_dir).encode(a.style_text)], dtype=torch.long)
    if a.speaker:
        cond["speaker"] = a.speaker
    elif a.ref_audio_path:
        cond["speaker_embedding"] = B.extract_speaker_embedding_from_audio(model, a.ref_audio_path, a.speaker_mel_path, a.speaker_mel_frames_path)[:, 0]
    opt = T.SamplingOptions(a.temperature, a.top_k, a.top_p, a.repetition_penalty, a.suppress_tail, a.subtalker_temperature, a.subtalker_top_k,
                            a.subtalker_top_p, _floats(a.subtalker_temp_by_group), _ints(a.subtalker_top_k_by_group), _floats(a.subtalker_top_p_by_group))
    gen = torch.Generator().manual_seed(a.seed)
    if a.streaming_decode and not a.skip_decode:
        if model.speech_decoder is None:
            raise SystemExit("streaming decode needs speech_tokenizer/ next to the model")
        chunks = []
        frames = model.stream(text_ids, lambda w: chunks.append(w.float().cpu()), a.max_frames, a.stream_chunk_frames, opt, gen, **cond)
        wave = torch.cat(chunks) if chunks else torch.zeros(0)
        os.makedirs(os.path.dirname(a.wav_path) or ".", exist_ok=True)
        media.save_wav(a.wav_path, wave, 24000)
        print(f"frames={frames} saved_audio={a.wav_path} samples={wave.numel()}")
        return 0
    codes, lengths = model.generate_from_text(text_ids, a.max_frames, opt, gen, **cond)
    n = max(1, lengths[0])
    os.makedirs(os.path.dirname(a.codes_path) or ".", exist_ok=True)
    with open(a.codes_path, "w", encoding="utf-8") as f:
        f.write(B.format_code_rows(codes[0, :n].reshape(-1).tolist(), codes.shape[2]))
    print(f"frames={n} saved_codes={a.codes_path}")
    if a.skip_decode:
        return 0
    if model.speech_decoder is None:
        raise SystemExit("no speech_tokenizer/ next to the model: pass --skip-decode or add the tokenizer directory")
    samples = B.decode_codes_to_wav(model.speech_decoder, a.codes_path, a.wav_path, num_code_groups=codes.shape[2])
    print(f"saved_audio={a.wav_path} samples={samples}")
    return 0


def run_kitten(argv) -> int:
    from ..models import kitten_tts_io as KIO
    if len(argv) not in (4, 5):
        print("Usage: run_tts kitten <model_dir_or_repo> <phonemes> <voice> <out_audio> [speed]", file=sys.stderr)
        return 1
    source, phonemes, voice, out_path = argv[:4]
    try:
        speed = float(argv[4]) if len(argv) == 5 else 1.0
    except ValueError:
        print(f"Invalid speed: {argv[4]}", file=sys.stderr)
        return 1
    bundle = KIO.load_from_pretrained(source, log=print)
    out = bundle.synthesize_phonemes_to_file(phonemes, voice, out_path, speed)
    print(f"saved_audio={out_path}")
    print(f"alignment_frames={out.alignment_frames}")
    print(f"pred_durations={out.pred_durations}")
    print(f"audio_shape={list(out.audio.shape)}")
    return 0


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if not argv or argv[0] not in ("qwen3tts", "kitten"):
        print("usage: run_tts {qwen3tts,kitten} ...", file=sys.stderr)
        return 1
    return run_qwen(argv[1:]) if argv[0] == "qwen3tts" else run_kitten(argv[1:])


if __name__ == "__main__":
    sys.exit(main())
