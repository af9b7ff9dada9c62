// Golden-vector dumper for the cached attention paths of relux.  NOT compiled in this repository's build image (there
// is no Go toolchain there); it is for a maintainer who has relux and Go:
//
//	cp relux_golden_dump_test.go  <relux>/internal/transformer/
//	cd <relux> && RELUX_GOLDEN_OUT=/tmp/relux_go_golden.json go test ./internal/transformer -run TestDumpReluxGolden
//	cp /tmp/relux_go_golden.json  <this repo>/tests/golden/
//
// tests/test_reference_golden_optional.py then compares the CPU oracle (FAITHFUL mode: the reference's behaviour with
// its cache-layout and position rules as they are) with these outputs bit for bit, which pins the oracle's
// restatement of MHA.forwardCached and MLA.forwardCached against a real relux run; the "sampler" section does the same
// for Sampler.Sample (tokens for recorded draws).
//
// Everything is generated from one 64-bit LCG so that the Python side can rebuild weights and inputs exactly:
//
//	state = state*6364136223846793005 + 1442695040888963407 (mod 2^64);  value = float32(int32(state >> 32)) / 2^31
//
// Weights are value * 0.25 rounded with BF16FromF32; inputs are the raw values.  Order of draws: for MHA Wq, Wk, Wv,
// Wo (row-major as stored), then the prompt x[8][64], then 4 single-token inputs; for MLA W_Q, W_DKV, W_UK, W_UV,
// W_KR, W_QR, W_O, then the prompt and the 4 single-token inputs.
package transformer

import (
	"encoding/json"
	"math"
	"math/rand"
	"os"
	"testing"
)

type goldenLCG uint64

func (s *goldenLCG) next() float32 {
	*s = *s*6364136223846793005 + 1442695040888963407
	return float32(int32(uint32(uint64(*s)>>32))) / 2147483648.0
}

func (s *goldenLCG) fillBF16(dst []uint16) {
	for i := range dst {
		dst[i] = BF16FromF32(s.next() * 0.25)
	}
}

func (s *goldenLCG) tensor(rows, cols int) *Tensor {
	d := make([]float32, rows*cols)
	for i := range d {
		d[i] = s.next()
	}
	return NewTensor(d, 1, rows, cols)
}

func goldenBits(t *Tensor) []uint32 {
	d, _ := t.ToF32()
	out := make([]uint32, len(d))
	for i, v := range d {
		out[i] = math.Float32bits(v)
	}
	return out
}

func TestDumpReluxGolden(t *testing.T) {
	path := os.Getenv("RELUX_GOLDEN_OUT")
	if path == "" {
		t.Skip("set RELUX_GOLDEN_OUT to the JSON file to write")
	}
	result := map[string]interface{}{"format": 1, "prompt_tokens": 8, "decode_steps": 4}

	// ---- MHA with GQA: dModel 64, 4 heads, 2 kv heads (head_dim 16), RoPE base 10000, maxSeqLen 64, causal ----
	{
		var g goldenLCG = 12345
		rope := NewRotaryEmbedding(16, 10000, 64)
		m := NewMHA(64, 4, 2, rope, true)
		g.fillBF16(m.Wq.Data)
		g.fillBF16(m.Wk.Data)
		g.fillBF16(m.Wv.Data)
		g.fillBF16(m.Wo.Data)
		m.SetMode(Inference)
		m.Cache = NewKVCacheSized(1, 64, 2, 16, BFloat16)
		m.LayerIdx = 0
		outs := [][]uint32{goldenBits(m.Forward(g.tensor(8, 64)))}
		for i := 0; i < 4; i++ {
			outs = append(outs, goldenBits(m.Forward(g.tensor(1, 64))))
		}
		result["mha"] = map[string]interface{}{"d_model": 64, "heads": 4, "kv_heads": 2, "seed": 12345, "outputs_f32_bits": outs}
	}

	// ---- MLA: dModel 64, 4 heads (head_dim 16), dC 32, dHR 8, maxSeqLen 64, RoPE base 10000, causal ----
	{
		var g goldenLCG = 54321
		m := NewMLA(64, 4, 32, 8, 64, 10000, true)
		g.fillBF16(m.W_Q.Data)
		g.fillBF16(m.W_DKV.Data)
		g.fillBF16(m.W_UK.Data)
		g.fillBF16(m.W_UV.Data)
		g.fillBF16(m.W_KR.Data)
		g.fillBF16(m.W_QR.Data)
		g.fillBF16(m.W_O.Data)
		m.SetMode(Inference)
		m.Cache = NewMLACache(1, 64, 32, 8)
		m.LayerIdx = 0
		outs := [][]uint32{goldenBits(m.Forward(g.tensor(8, 64)))}
		for i := 0; i < 4; i++ {
			outs = append(outs, goldenBits(m.Forward(g.tensor(1, 64))))
		}
		result["mla"] = map[string]interface{}{"d_model": 64, "heads": 4, "dC": 32, "dHR": 8, "seed": 54321, "outputs_f32_bits": outs}
	}

	// ---- Sampler.Sample: 6 settings x 8 rows of 500 logits (LCG values * 6), seed 777.  Two generators with the same
	// seed: one is consumed by Sample, the other records the draw Sample took, so the Python side needs no math/rand. ----
	{
		var g goldenLCG = 777
		settings := []Sampler{
			{Temperature: 1, TopP: 1},
			{Temperature: 0.7, TopP: 1},
			{Temperature: 1, TopK: 40, TopP: 1},
			{Temperature: 1, TopP: 0.9},
			{Temperature: 1, TopP: 1, MinP: 0.05},
			{Temperature: 1.3, TopK: 100, TopP: 0.85, MinP: 0.02, RepeatPenalty: 1.2, FrequencyPenalty: 0.2, PresencePenalty: 0.3, RepeatWindow: 16},
		}
		var cases []map[string]interface{}
		for si := range settings {
			s := settings[si]
			s.Rand = rand.New(rand.NewSource(int64(1000 + si)))
			shadow := rand.New(rand.NewSource(int64(1000 + si)))
			for row := 0; row < 8; row++ {
				logits := make([]float32, 500)
				for i := range logits {
					logits[i] = g.next() * 6
				}
				prev := make([]int, 24)
				for i := range prev {
					prev[i] = int((g.next() + 1) * 250)
				}
				draw := shadow.Float32()
				tok := s.Sample(logits, prev)
				cases = append(cases, map[string]interface{}{"setting": si, "draw_bits": math.Float32bits(draw), "token": tok})
			}
		}
		result["sampler"] = map[string]interface{}{"seed": 777, "vocab": 500, "rows_per_setting": 8, "prev_len": 24, "cases": cases}
	}

	b, err := json.Marshal(result)
	if err != nil {
		t.Fatal(err)
	}
	if err := os.WriteFile(path, b, 0644); err != nil {
		t.Fatal(err)
	}
}
