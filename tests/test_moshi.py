"""Moshi's temporal and depth transformers against Transformers on the same (tiny, random) weights."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from eredu_b200.models.moshi import MoshiConfig, MoshiLm

K = 3


def tiny(tmp_path):
    cfg = transformers.MoshiConfig(
        vocab_size=64, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, audio_vocab_size=17,
        max_position_embeddings=128, sliding_window=64, ffn_dim=64, num_codebooks=K,
        depth_decoder_config=dict(hidden_size=16, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2, ffn_dim=32,
                                  max_position_embeddings=K, sliding_window=K, input_size=32, audio_vocab_size=17, vocab_size=64,
                                  num_codebooks=K),
        audio_encoder_config=dict(model_type="mimi", hidden_size=32, num_filters=8, upsampling_ratios=[4, 2], codebook_size=16,
                                  codebook_dim=8, num_quantizers=K, vector_quantization_hidden_dimension=8, num_hidden_layers=1,
                                  num_attention_heads=4, num_key_value_heads=4, head_dim=8, intermediate_size=64, sliding_window=16,
                                  frame_rate=150.0, upsample_groups=32, sampling_rate=2400))
    torch.manual_seed(0)
    m = transformers.MoshiForConditionalGeneration(cfg).eval().float()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if not name.startswith("audio_encoder"):
                p.add_(torch.randn(p.shape, generator=g) * (0.1 if p.dim() == 1 else 0.05))
    m.save_pretrained(tmp_path, safe_serialization=True)
    return m


def test_temporal_and_depth_match_transformers(tmp_path):
    hf = tiny(tmp_path)
    lm = MoshiLm.load(tmp_path)
    cfg = lm.cfg
    assert isinstance(cfg, MoshiConfig) and cfg.num_codebooks == K and cfg.depth["hidden_size"] == 16 and cfg.sliding_window == 64
    g = torch.Generator().manual_seed(2)
    T = 20
    text = torch.randint(0, 64, (2, T), generator=g)
    spoken = torch.randint(0, 17, (2, K, T), generator=g)
    heard = torch.randint(0, 17, (2, K, T), generator=g)
    with torch.no_grad():
        out = hf(input_ids=text, moshi_audio_codes=spoken, user_audio_codes=heard)
    logits, hidden = lm.temporal(lm.embed_frame(text, spoken, heard))
    assert torch.allclose(logits, out.logits.float(), atol=2e-4), float((logits - out.logits).abs().max())
    assert torch.allclose(hidden, out.last_hidden_state, atol=2e-4)
    # incremental: a prefix, then one frame at a time, equals the full pass - also with a window shorter than the clip
    # (Transformers applies the window to its cache only, so that case is checked against this model's own full pass)
    lm.cfg.sliding_window = 12
    windowed, _ = lm.temporal(lm.embed_frame(text, spoken, heard))
    assert torch.allclose(windowed[:, :12], logits[:, :12], atol=1e-5) and not torch.allclose(windowed[:, 12:], logits[:, 12:], atol=1e-3)
    logits = windowed
    st: dict = {}
    x = lm.embed_frame(text, spoken, heard)
    parts = [lm.temporal(x[:, :7], st)[0]] + [lm.temporal(x[:, t:t + 1], st)[0] for t in range(7, T)]
    assert torch.allclose(torch.cat(parts, 1), logits, atol=1e-4) and st["pos"] == T
    assert st[0][0].shape[2] == 11                                     # the cache holds the window, not the clip
    # depth transformer, teacher forced: HF reads [text token, codebook 0 .. K-2] for one frame
    h = out.last_hidden_state[:, -1]
    frame_text, frame_audio = text[:, -1], spoken[:, :, -1]
    with torch.no_grad():
        want = hf.depth_decoder(input_ids=torch.cat((frame_text[:, None], frame_audio[:, :K - 1]), 1),
                                last_hidden_state=h[:, None]).logits
    got = lm.depth_logits(hidden[:, -1], frame_text, frame_audio)
    assert got.shape == want.shape == (2, K, 17) and torch.allclose(got, want.float(), atol=2e-4)
    # greedy generation of a frame feeds each choice to the next position
    toks = lm.depth_generate(hidden[:, -1], frame_text)
    again = lm.depth_logits(hidden[:, -1], frame_text, toks)
    assert toks.shape == (2, K) and torch.equal(again.argmax(-1), toks)
    picked = []
    lm.depth_generate(hidden[:, -1], frame_text, choose=lambda k, lg: picked.append(k) or lg.argmin(-1))
    assert picked == list(range(K))
    # missing streams (negative codes / None) contribute nothing
    x0 = lm.embed_frame(text, None, torch.full_like(heard, -1))
    assert torch.equal(x0, torch.nn.functional.embedding(text, lm.text_embed))


def test_realtime_session_delays_and_pipeline(tmp_path):
    from eredu_b200.codec import Mimi
    from eredu_b200.runtime.realtime import (RealtimeConfigError, RealtimeSampling, RealtimeSession, RealtimeSpeechConfig,
                                              SpeechPipeline)

    hf = tiny(tmp_path)
    lm = MoshiLm.load(tmp_path)
    speech = RealtimeSpeechConfig.for_moshi(lm.cfg)
    assert speech.audio_delays == (0, 1, 1, 0, 1, 1) and speech.max_audio_delay == 1 and speech.text_padding_token == 64
    for bad in (dict(total_audio_codebooks=6, input_audio_codebooks=2), dict(audio_delays=(0, 1)), dict(depth_audio_codebooks=4)):
        kw = dict(total_audio_codebooks=6, input_audio_codebooks=3, generated_audio_codebooks=3, depth_audio_codebooks=3,
                  text_padding_token=64, audio_padding_token=17, audio_delays=(0, 1, 1, 0, 1, 1))
        kw.update(bad)
        with pytest.raises(RealtimeConfigError):
            RealtimeSpeechConfig(**kw)
    with pytest.raises(RealtimeConfigError):
        RealtimeSampling(text_temperature=-1.0)
    greedy = RealtimeSampling(text_temperature=0.0, audio_temperature=0.0)
    sess = RealtimeSession(lm, speech, greedy)
    g = torch.Generator().manual_seed(3)
    heard = torch.randint(0, 16, (6, 1, K), generator=g)
    steps = [sess.step(heard[t]) for t in range(6)]
    assert steps[0].spoken_codes is None and all(s.spoken_codes is not None for s in steps[1:])
    # replay by hand: rows in delayed coordinates, teacher-forced through the full-sequence passes
    text_rows = [torch.tensor([64])] + [s.text_token for s in steps[:-1]]
    spoken_rows, heard_rows = [torch.full((1, K), 17)], [torch.full((1, K), 17)]
    state: dict = {}
    rows_generated = []
    for t in range(6):
        x = lm.embed_frame(text_rows[t][:, None], spoken_rows[t][:, :, None], heard_rows[t][:, :, None])
        logits, hidden = lm.temporal(x, state)
        tok = logits[:, -1].argmax(-1)
        assert torch.equal(tok, steps[t].text_token)
        row = lm.depth_generate(hidden[:, -1], tok)
        rows_generated.append(row)
        spoken_rows.append(row)
        h = torch.full((1, K), 17)
        h[:, 0] = heard[t][:, 0]                                   # semantic codebook: no delay
        if t >= 1:
            h[:, 1:] = heard[t - 1][:, 1:]                         # acoustic codebooks: one frame behind
        heard_rows.append(h)
    for t in range(1, 6):                                          # output frame t-1: codebook 0 of row t-1, the others of row t
        want = torch.cat((rows_generated[t - 1][:, :1], rows_generated[t][:, 1:]), 1)
        assert torch.equal(steps[t].spoken_codes, want)
    # seeded sampling is reproducible and differs from greedy decoding somewhere
    a = [RealtimeSession(lm, speech, RealtimeSampling(seed=4)).step(heard[0]).text_token for _ in range(2)]
    assert torch.equal(a[0], a[1])
    # PCM in, PCM out through the codec (Moshi's audio encoder weights live under audio_encoder.* in the same checkpoint)
    sd = {k[len("audio_encoder."):]: v for k, v in hf.state_dict().items() if k.startswith("audio_encoder.")}
    from eredu_b200.codec import MimiConfig

    codec = Mimi(MimiConfig.from_dict(hf.config.audio_encoder_config.to_dict()), sd.__getitem__)
    pipe = SpeechPipeline(RealtimeSession(lm, speech, greedy), codec)
    F_ = codec.cfg.frame_size
    assert pipe.feed(torch.randn(1, 1, F_ - 3, generator=g)) is None             # not a whole frame yet
    assert pipe.feed(torch.randn(1, 1, 3, generator=g)) is None                   # first frame: output still inside the delay
    out = pipe.feed(torch.randn(1, 1, 3 * F_, generator=g))
    assert out.shape == (1, 1, 3 * F_) and len(pipe.text_tokens) == 4 and torch.isfinite(out).all()


def test_realtime_scheduler_is_fair_and_tracks_deadlines():
    from eredu_b200.runtime.realtime import RealtimeError, RealtimeScheduler

    class Fake:
        def __init__(self, name):
            self.name, self.seen = name, []

        def step(self, inp):
            self.seen.append(inp)
            return f"{self.name}:{inp}"

    now = [0.0]
    sch = RealtimeScheduler(max_queue_per_request=4, clock=lambda: now[0])
    a, b = sch.register_request(Fake("a")), sch.register_request(Fake("b"))
    for i in range(3):
        sch.enqueue(a, i)
    sch.enqueue(b, 10, deadline=5.0)
    sch.enqueue(b, 11, deadline=0.5)
    now[0] = 1.0
    done = sch.run_bounded(3)
    assert [d.output for d in done] == ["a:0", "b:10", "a:1"] and not any(d.late for d in done)
    rest = sch.run_queued()
    assert [d.output for d in rest] == ["b:11", "a:2"] and rest[0].late and not rest[1].late
    rep = sch.report()
    assert rep["steps_run"] == 5 and rep["requests"][b]["missed_deadlines"] == 1 and rep["requests"][a]["completed"] == 3
    with pytest.raises(RealtimeError):
        sch.enqueue_batch([(a, i) for i in range(5)])                            # over the limit: nothing is queued
    assert sch.queued_for_request(a) == 0
    sch.enqueue(a, 7)
    with pytest.raises(RealtimeError):
        sch.finish_request(a)                                                     # work still queued
    sch.cancel_request(a)
    assert sch.request_status(a) == "cancelled" and sch.queued_for_request(a) == 0 and sch.run_queued() == []
    sch.finish_request(b)
    with pytest.raises(RealtimeError):
        sch.enqueue(b, 1)
    sch.forget_terminal_request(a)
    assert sch.request_status(a) is None and sch.request_status(b) == "finished"


def test_inspection_names_the_speech_loaders(tmp_path):
    from eredu_b200.runtime.plan import inspect_artifact

    tiny(tmp_path)
    rep = inspect_artifact(tmp_path)
    assert rep.model_type == "moshi" and not rep.is_loadable and rep.tensor_count > 0
    assert [i.code for i in rep.issues] == ["speech_model"] and "MoshiLm.load" in rep.issues[0].message
    (tmp_path / "model.safetensors").unlink()
    import safetensors.torch

    safetensors.torch.save_file({"decoder.model.norm.weight": torch.zeros(4)}, str(tmp_path / "model.safetensors"))
    codes = [i.code for i in inspect_artifact(tmp_path).issues]
    assert codes.count("missing_tensor") == 3 and codes[-1] == "speech_model"
