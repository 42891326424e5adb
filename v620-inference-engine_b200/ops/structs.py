"""ctypes mirrors of the runtime structs in ``csrc/runtime.h`` (same field order and types)."""
import ctypes as C

P = C.c_void_p


class QwDims(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "ranks", "rank", "H", "hc", "hc_rank", "SH", "n_layers", "vocab", "vocab_l",
        "QL", "KVL", "IH", "proj_qsa", "KL", "VL", "proj_gdn",
        "E", "E_l", "e_first", "top_k", "F", "SF",
        "ple_layer", "ple_kv", "ngram_heads", "ngram_dim", "ple_taps", "ple_dil",
        "idx_ratio", "idx_topk", "nsplit", "max_rows",
        "slots", "max_pages", "n_dev_pages", "ck_cap", "score_cap")] + [("eps", C.c_float)]


class QwHc(C.Structure):
    _fields_ = [("w1", P), ("Wd", P), ("Wu", P), ("n_inj", C.c_int), ("pad_", C.c_int)]


class QwLayer(C.Structure):
    _fields_ = [("is_qsa", C.c_int), ("state_index", C.c_int), ("attn_hc", QwHc), ("mlp_hc", QwHc),
                ("Wproj", P), ("Wout", P), ("cw", P), ("A_log", P), ("dt_bias", P), ("gdn_norm", P),
                ("qn1", P), ("kn1", P), ("iqn1", P), ("ikn1", P),
                ("Wrs", P), ("w13", P), ("s13", P), ("w2", P), ("s2", P), ("Wsd", P)]


class QwPle(C.Structure):
    _fields_ = [("Wkv", P), ("nk1", P), ("nq1", P), ("nc1", P), ("cw", P), ("shards", P), ("scales", P),
                ("rows_per_shard", C.c_longlong), ("rows", C.c_longlong), ("layout", C.c_int), ("enabled", C.c_int)]


class QwMtp(C.Structure):
    _fields_ = [("enabled", C.c_int), ("pad_", C.c_int), ("layer", QwLayer), ("final_hc", QwHc), ("fc_h", P), ("fc_e", P),
                ("nh1", P), ("ne1", P), ("hn", P), ("en", P), ("fh", P), ("fe", P)]


class QwState(C.Structure):
    _fields_ = [(n, P) for n in ("k_dev", "v_dev", "k_host", "v_host", "ck", "raw_ring", "gdn_S", "gdn_ring",
                                 "ple_ring", "page_table")]


BUFFER_FIELDS = ("X", "y", "send", "red", "bin", "proj", "inj_a", "inj_b", "partial", "out_a", "out_b", "o",
                 "qkv", "decay", "beta", "q", "iq", "scores", "sel", "sel_n", "pm", "pl", "pacc", "rs",
                 "pair_expert", "pair_w", "sh_h", "moe_h", "ple_e", "ple_kv", "ple_send", "ple_red", "ple_gv",
                 "ple_nc", "logits", "amax_val", "amax_idx", "lse_max", "lse_sum", "gdn_save", "hidden_out", "X2", "ticket")


class QwBuffers(C.Structure):
    _fields_ = [(n, P) for n in BUFFER_FIELDS]


class QwRows(C.Structure):
    _fields_ = [("M", C.c_int), ("max_groups", C.c_int), ("tokens", P), ("slot", P), ("pos", P), ("run_start", P),
                ("run_len", P), ("ctx3", P)]


COMM_FN = C.CFUNCTYPE(None, P, C.c_int, C.c_int, P, P, C.c_int, C.c_int, P)


class QwModel(C.Structure):
    _fields_ = [("d", QwDims), ("layers", C.POINTER(QwLayer)), ("final_hc", QwHc), ("ple", QwPle), ("embed", P),
                ("lm_head", P), ("st", QwState), ("b", QwBuffers), ("comm", COMM_FN), ("comm_user", P),
                ("p2p", P), ("amax_pairs", P), ("off_amax", C.c_longlong), ("off_bin", C.c_longlong), ("mtp", QwMtp),
                ("mtp_hid", P), ("off_mtp_hid", C.c_longlong), ("off_logits", C.c_longlong), ("logits_ld", C.c_int),
                ("pad2_", C.c_int)]


class QwP2P(C.Structure):
    _fields_ = [("peer", P * 8), ("ranks", C.c_int), ("rank", C.c_int), ("base", P), ("off_flags", C.c_longlong * 4),
                ("off_recv", C.c_longlong * 4), ("slot_bytes", C.c_longlong * 4), ("off_bin", C.c_longlong),
                ("off_amax", C.c_longlong)]


# ---- token-major prefill runtime (csrc/prefill_rt.h, csrc/tp.cuh) -------------------------------------------------
TP_KINDS = 6
TP_SSQ, TP_DOWN, TP_BIN, TP_RS, TP_SMALL, TP_WIDE = range(6)


class QwTp(C.Structure):
    _fields_ = [("peer", P * 8), ("ranks", C.c_int), ("rank", C.c_int), ("off_flags", C.c_longlong),
                ("off_buf", C.c_longlong * 6), ("part_bytes", C.c_longlong * 6), ("ticket", P), ("seq", C.c_uint * 6),
                ("spin_limit", C.c_uint), ("pad_", C.c_int)]


PREFILL_PTR_FIELDS = (
    "X", "xn", "d", "u", "inj_a", "inj_b", "g", "bin", "proj", "o", "out_a", "out_b", "qkv", "decay", "beta",
    "q", "iq", "scores", "sel", "sel_n", "rs", "pe", "pw", "sh_h", "sd", "xperm", "h13", "h", "y", "inv", "src_token",
    "t13", "t2", "gdn_scratch", "ple_e", "ple_kv", "ple_send", "ple_red", "ple_gv", "ple_nc",
    "Xm", "hn", "en", "fh", "fe", "mtp_ssq", "mtp_tok", "hid_out", "amax16",
    "tokens", "slot", "pos", "run_start", "run_len", "ctx3", "m_slot", "m_pos", "m_run_start", "m_run_len",
    "over_rows", "over_emb", "stage_k", "stage_v")
PREFILL_INT_FIELDS = ("cap", "hc_ld", "hc_ksplit", "nrs_ld", "proj_ld", "o_ld", "ple_ld", "max_tiles")


class QwPrefillBufs(C.Structure):
    _fields_ = [(n, P) for n in PREFILL_PTR_FIELDS] + [(n, C.c_int) for n in PREFILL_INT_FIELDS] + \
               [("gdn_scratch_lane", C.c_longlong)]


PREFILL_HOOK = C.CFUNCTYPE(None, P, C.c_int, C.c_int, P, C.c_int, C.c_int, C.c_int)


class QwPrefillJob(C.Structure):
    _fields_ = [("md", C.POINTER(QwModel)), ("b", C.POINTER(QwPrefillBufs)), ("tp", P * 2), ("stream", P * 2),
                ("T", C.c_int), ("lanes", C.c_int), ("base", C.c_int), ("want_logits", C.c_int), ("layer_limit", C.c_int),
                ("mtp_rows", C.c_int), ("mtp_base", C.c_int), ("has_pending", C.c_int), ("n_over", C.c_int), ("n0", C.c_int),
                ("hook", PREFILL_HOOK), ("hook_user", P), ("slot", C.c_int), ("pad_", C.c_int)]


def check_prefill_structs(lib) -> None:
    """The C side's struct sizes must equal the mirrors' (a mismatch means the two field lists have drifted apart)."""
    lib.qwrt_prefill_sizes.restype = C.c_longlong
    lib.qwrt_prefill_sizes.argtypes = [C.c_int]
    for which, cls in ((0, QwPrefillBufs), (1, QwPrefillJob), (2, QwTp)):
        want, have = int(lib.qwrt_prefill_sizes(which)), C.sizeof(cls)
        if want != have:
            raise RuntimeError(f"{cls.__name__}: ctypes mirror is {have} bytes, the library's struct {want}")
