// Plan -> stage program. This is the engine's code generator: where the
// reference emits CUDA source per plan (ark/codegen.cpp:79-429) this emits a
// table of stages for the prebuilt sm_100a loop kernel.
//
// What is kept from the plan: the processor ranges (which CTAs run what, and
// therefore which groups run concurrently), the order of processor groups,
// the barrier rule between them (codegen.cpp:109-158) and the task ranges.
// What is not kept: the mapping of task ids to warps/shared-memory slots
// inside a CTA (WarpRange, SramRange, NumWarps, SramBytes are validated and
// otherwise ignored) — here a whole CTA works on one stage at a time and an
// op's work is split over the CTAs of its range by the op's own kernel.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>
#include <sstream>

#include "plan.hpp"

namespace arkb {

namespace {

constexpr size_t kFullSmemBytes = 208 * 1024;  // operand ring (192 KiB) + epilogue staging (16 KiB) of the tensor-core matmul

struct Lowerer {
    const Plan &plan;
    const Layout &lay;
    const LowerEnv &env;
    Program prog;
    std::map<std::tuple<int64_t, int64_t, int64_t>, int> sync_ids;
    int oneshot_ord = 0;

    Lowerer(const Plan &p, const Layout &l, const LowerEnv &e) : plan(p), lay(l), env(e) {}

    // ---- helpers ---------------------------------------------------------------
    char *tensor_ptr(const TensorDesc &t) const {
        const BufferInfo &b = lay.buffers.at(t.buffer_id);
        if (!b.resolved) throw Error(E_PLAN, "buffer " + std::to_string(b.id) + " has no address");
        int r = (b.rank == -1) ? env.rank : b.rank;
        if (r < 0 || r >= env.nranks || !env.arena[r]) throw Error(E_PLAN, "tensor on unmapped rank " + std::to_string(r));
        int64_t es[4], org;
        t.elem_strides(es, org);
        return env.arena[r] + b.offset + (size_t)org * dtype_size(t.dtype);
    }

    // View of `t` broadcast to the 4-D shape `osh` (NumPy rules on dims4).
    TRef make_ref(const TensorDesc &t, const std::vector<int64_t> *osh = nullptr) const {
        TRef r;
        std::memset(&r, 0, sizeof(r));
        r.ptr = tensor_ptr(t);
        r.dtype = t.dtype;
        int64_t es[4], org;
        t.elem_strides(es, org);
        auto sh = t.shape4();
        for (int i = 0; i < 4; ++i) {
            int64_t target = osh ? (*osh)[i] : sh[i];
            if (sh[i] != target && sh[i] != 1) throw Error(E_MODEL, "shapes do not broadcast");
            r.shape[i] = (int32_t)target;
            r.stride[i] = (sh[i] == 1 && target != 1) ? 0 : es[i];
            if (sh[i] == 1) r.stride[i] = (target == 1) ? es[i] : 0;
        }
        r.contiguous = t.dense() ? 1 : 0;
        return r;
    }

    // fp32 value after a round trip through the storage type (round to nearest even)
    static float round_to_dtype(float v, int dt) {
        uint32_t x;
        std::memcpy(&x, &v, 4);
        if (dt == DT_BF16) {
            if ((x & 0x7f800000u) != 0x7f800000u) x += 0x7fffu + ((x >> 16) & 1u);
            x &= 0xffff0000u;
            std::memcpy(&v, &x, 4);
            return v;
        }
        if (dt == DT_F16) {
            const uint32_t sign = x & 0x80000000u;
            const int32_t e = (int32_t)((x >> 23) & 0xff) - 127;
            if (e > 15) return v;                 // overflow/inf/nan: leave to the device conversion
            if (e < -25 || (e == -25 && (x & 0x7fffffu) == 0)) { x = sign; std::memcpy(&v, &x, 4); return v; }
            if (e == -25) { x = sign | 0x33800000u; std::memcpy(&v, &x, 4); return v; }  // rounds up to 2^-24
            // keep 10 mantissa bits (fewer for subnormal halves)
            const int drop = e >= -14 ? 13 : 13 + (-14 - e);
            const uint32_t mant = x & 0x7fffffffu;
            const uint32_t half = 1u << (drop - 1), mask = (1u << drop) - 1;
            uint32_t r = mant & ~mask;
            const uint32_t rem = mant & mask;
            if (rem > half || (rem == half && (r >> drop & 1u))) r += (1u << drop);
            x = sign | r;
            std::memcpy(&v, &x, 4);
            return v;
        }
        return v;
    }

    static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

    Stage new_stage(int kind, const Range &proc) {
        Stage s;
        std::memset(&s, 0, sizeof(s));
        s.kind = kind;
        s.proc_b = (int32_t)proc.b;
        s.proc_e = (int32_t)proc.e;
        s.proc_s = (int32_t)proc.s;
        return s;
    }
    // ---- what the stage being built touches (see StageAccess) ---------------------------------
    StageAccess acc;
    void acc_begin() {
        acc = StageAccess();
        acc.opaque = false;
    }
    static std::pair<uintptr_t, uintptr_t> span_of(const void *p, size_t bytes) {
        const uintptr_t b = reinterpret_cast<uintptr_t>(p);
        return {b, b + bytes};
    }
    std::pair<uintptr_t, uintptr_t> span_of(const TensorDesc &t) const {
        int64_t es[4], org;
        t.elem_strides(es, org);
        auto sh = t.shape4();
        int64_t last = 0;
        for (int i = 0; i < 4; ++i) last += (sh[i] - 1) * es[i];
        return span_of(tensor_ptr(t), (size_t)(last + 1) * dtype_size(t.dtype));
    }
    void rd(const TensorDesc &t) { acc.reads.push_back(span_of(t)); }
    // a read operand the stage streams once (weights, caches): may be fetched into L2 ahead of time if nothing writes it
    void rd_streamed(const TensorDesc &t) {
        auto sp = span_of(t);
        acc.reads.push_back(sp);
        if (sp.second - sp.first >= 32 * 1024 && (t.buffer_rank == -1 || t.buffer_rank == env.rank))
        {
            const uintptr_t b = (sp.first + 15) & ~(uintptr_t)15, e = sp.second & ~(uintptr_t)15;  // bulk prefetch wants 16-byte units
            acc.streamed.push_back({reinterpret_cast<const void *>(b), (size_t)(e - b), t.buffer_id});
        }
    }
    void wr(const TensorDesc &t) { acc.writes.push_back(span_of(t)); }
    void rd_raw(const void *p, size_t bytes) { if (p && bytes) acc.reads.push_back(span_of(p, bytes)); }
    void wr_raw(const void *p, size_t bytes) { if (p && bytes) acc.writes.push_back(span_of(p, bytes)); }

    void push(const Stage &s, const std::string &note) {
        prog.stages.push_back(s);
        prog.access.push_back(acc);
        acc = StageAccess();  // opaque until a lowering function says what its stage touches
        std::ostringstream os;
        os << "[" << s.proc_b << "," << s.proc_e << (s.proc_s != 1 ? "," + std::to_string(s.proc_s) : "") << ") " << note;
        prog.notes.push_back(os.str());
    }

    void emit_sync(const Range &r) {
        if (r.count() <= 0) return;
        auto key = std::make_tuple(r.b, r.e, r.s);
        auto it = sync_ids.find(key);
        int id;
        if (it == sync_ids.end()) {
            id = (int)sync_ids.size();
            if (id >= kMaxSyncGroups - 1) throw Error(E_UNSUPPORTED, "too many distinct processor ranges need a barrier");
            sync_ids[key] = id;
        } else {
            id = it->second;
        }
        Stage s = new_stage(SK_SYNC, r);
        s.sync_group = id;
        s.sync_count = (int32_t)r.count();
        s.sync_ord = ++prog.syncs_per_iter[id];
        push(s, "sync group " + std::to_string(id) + " #" + std::to_string(s.sync_ord));
    }

    static bool full_range(const Range &tr, int64_t num_tasks) { return tr.b == 0 && tr.s == 1 && tr.e >= num_tasks; }

    static int64_t config_int(const OpDesc &op, const char *key, int64_t dflt) {
        return op.config.is_object() && op.config.contains(key) ? op.config.at(key).as_int() : dflt;
    }

    int64_t num_tasks(const OpDesc &op) const {
        if (op.config.is_object() && op.config.contains("NumTasks")) return op.config.at("NumTasks").as_int();
        return 1;
    }

    // ---- elementwise -----------------------------------------------------------
    static int ewise_code(const std::string &t) {
        static const std::map<std::string, int> m = {
            {"Copy", EW_COPY}, {"Gelu", EW_GELU}, {"Exp", EW_EXP}, {"Relu", EW_RELU}, {"Rsqrt", EW_RSQRT},
            {"Sigmoid", EW_SIGMOID}, {"Sqrt", EW_SQRT}, {"Cast", EW_CAST}, {"Add", EW_ADD}, {"Sub", EW_SUB},
            {"Mul", EW_MUL}, {"Div", EW_DIV}, {"ScalarAssign", EW_SCALAR_ASSIGN}, {"ScalarAdd", EW_SCALAR_ADD},
            {"ScalarMul", EW_SCALAR_MUL}, {"Rope", EW_ROPE}, {"Silu", EW_SILU}};
        auto it = m.find(t);
        return it == m.end() ? -1 : it->second;
    }

    void lower_ewise(const OpDesc &op, const Range &proc, const TaskGroup &tg) {
        const int code = ewise_code(op.type);
        const bool binary = (code >= EW_ADD && code <= EW_DIV) || code == EW_ROPE;
        const bool has_in = code != EW_SCALAR_ASSIGN;
        const bool partial = !full_range(tg.task_range, num_tasks(op));
        const TensorDesc &out = op.results.at(0);
        if ((has_in && op.reads.size() < (binary ? 2u : 1u))) throw Error(E_MODEL, op.type + ": missing operand");
        Stage s = new_stage(SK_EWISE, proc);
        EwiseArgs &a = s.ew;
        acc_begin();
        wr(out);
        if (has_in) rd(op.reads[0]);
        if (binary) rd(op.reads[1]);
        auto osh = out.shape4();
        a.out = make_ref(out);
        if (has_in) a.in0 = make_ref(op.reads[0], &osh);
        if (binary) a.in1 = make_ref(op.reads[1], &osh);
        a.op = code;
        bool same = has_in ? (op.reads[0].shape4() == osh) : true;
        if (binary) same = same && (op.reads[1].shape4() == osh);
        // Collapse adjacent dimensions that every operand walks contiguously (or broadcasts
        // together), so that e.g. [N,C,H,W] + [1,1,1,W] is walked as [rows, W] with one division.
        if (partial) {
            // only the tiles of this task group: the walk keeps the 4-D form the task ids refer to
            if (!op.config.is_object() || !op.config.contains("Tile")) throw Error(E_PLAN, op.type + ": a partial TaskRange needs the Tile of the tasks");
            auto tile = op.config.at("Tile").as_int_vec();
            if (tile.size() != 2 || tile[0] <= 0 || tile[1] <= 0) throw Error(E_PLAN, "Tile should have 2 positive elements");
            a.task_b = (int32_t)tg.task_range.b;
            a.task_e = (int32_t)tg.task_range.e;
            a.task_s = (int32_t)tg.task_range.s;
            a.tile_h = (int32_t)tile[0];
            a.tile_w = (int32_t)tile[1];
            a.tiles_h = (int32_t)((osh[2] + tile[0] - 1) / tile[0]);
            a.tiles_w = (int32_t)((osh[3] + tile[1] - 1) / tile[1]);
        } else {
            TRef *refs[3] = {&a.out, has_in ? &a.in0 : nullptr, binary ? &a.in1 : nullptr};
            int64_t shp[4] = {osh[0], osh[1], osh[2], osh[3]};
            bool changed = true;
            while (changed) {
                changed = false;
                for (int i = 2; i >= 0; --i) {
                    if (shp[i] == 1) continue;
                    if (shp[i + 1] == 1) {  // empty slot below: move the dimension down
                        for (auto r : refs)
                            if (r) {
                                r->stride[i + 1] = r->stride[i];
                                r->stride[i] = 0;
                            }
                        shp[i + 1] = shp[i];
                        shp[i] = 1;
                        changed = true;
                        continue;
                    }
                    bool ok = true;
                    for (auto r : refs)
                        if (r && r->stride[i] != r->stride[i + 1] * shp[i + 1]) ok = false;
                    if (!ok) continue;
                    for (auto r : refs)
                        if (r) r->stride[i] = 0;
                    shp[i + 1] *= shp[i];
                    shp[i] = 1;
                    changed = true;
                }
            }
            for (auto r : refs)
                if (r)
                    for (int i = 0; i < 4; ++i) r->shape[i] = (int32_t)shp[i];
            osh = {shp[0], shp[1], shp[2], shp[3]};
        }
        // the scalar is rounded to the tensor's storage type first, as the reference's
        // host baselines do with T(factor) (ark/ops/ops_scalar_test.cpp:11-62)
        if (code == EW_SCALAR_ASSIGN) a.scalar = round_to_dtype((float)op.arg_float("Value"), out.dtype);
        if (code == EW_SCALAR_ADD || code == EW_SCALAR_MUL) a.scalar = round_to_dtype((float)op.arg_float("Factor"), out.dtype);
        const int idt = has_in ? op.reads[0].dtype : out.dtype;
        if (binary && op.reads[1].dtype != idt) throw Error(E_MODEL, op.type + ": operand data types differ");
        const bool convert = (code == EW_CAST) || idt != out.dtype;
        const bool integer = !(idt == DT_F32 || idt == DT_F16 || idt == DT_BF16);
        if (!convert && integer && !(code == EW_COPY || (code >= EW_ADD && code <= EW_DIV) || code == EW_SCALAR_ASSIGN ||
                                     code == EW_SCALAR_ADD || code == EW_SCALAR_MUL || code == EW_RELU))
            throw Error(E_UNSUPPORTED, op.type + ": not defined on integer tensors");
        if (!convert && integer && code != EW_COPY) {  // the scalar in the tensor's own arithmetic: T(factor), truncated
            if (code == EW_SCALAR_ASSIGN) a.scalar = (float)(int64_t)op.arg_float("Value");
            if (code == EW_SCALAR_ADD || code == EW_SCALAR_MUL) a.scalar = (float)(int64_t)op.arg_float("Factor");
        }
        int V = convert ? 4 : (int)(16 / dtype_size(out.dtype));
        if (code == EW_COPY && !convert) V = (int)(16 / dtype_size(out.dtype));
        const int64_t nelem = out.nelems();
        bool dense = out.dense() && (!has_in || op.reads[0].dense()) && (!binary || op.reads[1].dense());
        auto ptr_ok = [&](const TRef &r, int dt) {
            size_t bytes = (size_t)V * dtype_size(dt);
            size_t al = bytes > 16 ? 16 : bytes;
            return (reinterpret_cast<uintptr_t>(r.ptr) % al) == 0;
        };
        a.flat = (same && dense) ? 1 : 0;
        bool vec_ok = ptr_ok(a.out, out.dtype) && (!has_in || a.in0.stride[3] == 0 || ptr_ok(a.in0, idt)) &&
                      (!binary || a.in1.stride[3] == 0 || ptr_ok(a.in1, idt));
        if (a.flat) {
            vec_ok = vec_ok && (nelem % V == 0);
        } else {
            vec_ok = vec_ok && (osh[3] % V == 0);
            auto strides_ok = [&](const TRef &r) {
                if (r.stride[3] != 0 && r.stride[3] != 1) return false;
                if (r.stride[3] == 0) return true;  // broadcast along W: read as one scalar per unit
                for (int i = 0; i < 3; ++i)
                    if (r.stride[i] % V) return false;
                return true;
            };
            vec_ok = vec_ok && strides_ok(a.out) && (!has_in || strides_ok(a.in0)) && (!binary || strides_ok(a.in1));
        }
        if (code == EW_ROPE && !vec_ok && (osh[3] % 2)) throw Error(E_MODEL, "Rope needs an even innermost dimension");
        if (code == EW_ROPE && !vec_ok) {
            // pairs must stay together: fall back to 2-element units via the scalar walker is not
            // possible, so require vectorisable layouts
            throw Error(E_UNSUPPORTED, "Rope needs 16-byte aligned rows");
        }
        a.vec = vec_ok ? V : 1;
        if (partial) {
            a.vec = 1;
            a.flat = 0;
        }
        if (int64_t slots = config_int(op, "IterSlots", 1); slots > 1) {
            // ring of buffers walked by the iteration number (streaming input / output of a resident kernel)
            if (code != EW_COPY || convert) throw Error(E_UNSUPPORTED, op.type + ": IterSlots is for Copy between tensors of one type");
            a.iter_slots = (int32_t)slots;
            a.in_iter_bytes = config_int(op, "InIterStride", 0) * (int64_t)dtype_size(idt);
            a.out_iter_bytes = config_int(op, "OutIterStride", 0) * (int64_t)dtype_size(out.dtype);
            if (a.vec > 1 && (a.in_iter_bytes % 16 || a.out_iter_bytes % 16)) a.vec = 1;
        }
        if (a.flat) a.n_units = nelem / a.vec;
        else a.n_units = osh[0] * osh[1] * osh[2] * ((osh[3] + a.vec - 1) / a.vec);
        if (a.iter_slots > 1) {
            acc.opaque = true;  // the ring slots move with the iteration number
        } else if (a.flat && !convert && code != EW_ROPE && !(integer && code != EW_COPY)) {
            acc.aligned_units = a.n_units;
            acc.aligned_unit_bytes = (int)(a.vec * dtype_size(out.dtype));
        }
        push(s, op.type + " " + op.name + " units=" + std::to_string(a.n_units) + " vec=" + std::to_string(a.vec) +
                    (a.flat ? " flat" : " strided") +
                    (partial ? " tasks [" + std::to_string(a.task_b) + "," + std::to_string(a.task_e) + (a.task_s != 1 ? "," + std::to_string(a.task_s) : "") + ")" : ""));
    }

    // ---- reduce ------------------------------------------------------------------
    void lower_reduce(const OpDesc &op, const Range &proc, const TaskGroup &tg) {
        const bool partial = !full_range(tg.task_range, num_tasks(op));
        const TensorDesc &in = op.reads.at(0);
        TensorDesc out = op.results.at(0);
        int axis = (int)op.arg_int("Axis");
        const bool keep = op.arg_bool("KeepDim");
        const int nd = (int)in.shape.size();
        if (axis < 0) axis += nd;
        if (axis < 0 || axis >= nd) throw Error(E_MODEL, "invalid reduction axis");
        if (!keep) {  // re-insert the reduced dim (ark/ops/ops_reduce.cpp:93-98)
            out.shape.insert(out.shape.begin() + axis, 1);
            out.strides.insert(out.strides.begin() + axis, 1);
            out.offsets.insert(out.offsets.begin() + axis, 0);
            out.padded.insert(out.padded.begin() + axis, 1);
        }
        const int ax4 = axis + 4 - nd;
        if (in.dtype != out.dtype) throw Error(E_MODEL, "reduce: data types differ");
        if (!(in.dtype == DT_F32 || in.dtype == DT_F16 || in.dtype == DT_BF16))
            throw Error(E_UNSUPPORTED, "reduce: floating-point tensors only");
        Stage s = new_stage(SK_REDUCE, proc);
        ReduceArgs &a = s.rd;
        acc_begin();
        rd(in);
        wr(out);
        a.in = make_ref(in);
        a.out = make_ref(out);
        a.op = op.type == "ReduceSum" ? RD_SUM : op.type == "ReduceMax" ? RD_MAX : RD_MEAN;
        a.axis = ax4;
        const int V = (int)(16 / dtype_size(in.dtype));
        bool ok = aligned16(a.in.ptr) && a.in.stride[3] == 1;
        for (int i = 0; i < 3; ++i) ok = ok && (a.in.stride[i] % V == 0);
        if (ax4 != 3) {
            ok = ok && aligned16(a.out.ptr) && (in.shape4()[3] % V == 0) && a.out.stride[3] == 1;
            for (int i = 0; i < 3; ++i) ok = ok && (a.out.stride[i] % V == 0);
        }
        a.vec = ok ? V : 1;
        if (partial) {
            // a task is one output element (ark/ops/ops_reduce.cpp: NumTasks = elements of the result)
            if (num_tasks(op) != out.nelems()) throw Error(E_UNSUPPORTED, op.type + ": a partial TaskRange needs one task per output element");
            a.partial = 1;
            a.task_b = tg.task_range.b; a.task_e = std::min<int64_t>(tg.task_range.e, out.nelems()); a.task_s = std::max<int64_t>(1, tg.task_range.s);
            acc.opaque = false;
        }
        push(s, op.type + " " + op.name + " axis=" + std::to_string(ax4) + " vec=" + std::to_string(a.vec) +
                    (partial ? " tasks [" + std::to_string(a.task_b) + "," + std::to_string(a.task_e) + (a.task_s != 1 ? "," + std::to_string(a.task_s) : "") + ")" : ""));
    }

    // ---- fused row operators (engine extensions) -----------------------------------------
    void lower_rowop(const OpDesc &op, const Range &proc, const TaskGroup *tg = nullptr) {
        const TensorDesc &in = op.reads.at(0);
        const TensorDesc &out = op.results.at(0);
        Stage s = new_stage(SK_ROWOP, proc);
        RowOpArgs &a = s.ro;
        acc_begin();
        for (auto &t : op.reads) rd(t);
        for (auto &t : op.results) wr(t);
        for (auto &t : op.writes) wr(t);
        a.op = op.type == "RMSNorm" ? RO_RMSNORM : op.type == "LayerNorm" ? RO_LAYERNORM : RO_SOFTMAX;
        a.dtype = in.dtype;
        auto sh = in.shape4();
        auto ist = in.strides4();
        auto ost = out.strides4();
        a.cols = sh[3];
        a.rows = sh[0] * sh[1] * sh[2];
        a.in_ld = ist[3];
        a.out_ld = ost[3];
        // rows must be uniformly spaced: leading dims dense over H (and C, N)
        auto rows_uniform = [&](const TensorDesc &t) {
            auto s4 = t.shape4();
            auto st4 = t.strides4();
            auto of4 = t.offsets4();
            (void)of4;
            return (s4[0] * s4[1] == 1 || st4[2] == s4[2]) && (s4[0] == 1 || st4[1] == s4[1]);
        };
        if (!rows_uniform(in) || !rows_uniform(out)) throw Error(E_UNSUPPORTED, op.type + ": rows must be evenly spaced");
        a.in = tensor_ptr(in);
        a.out = tensor_ptr(out);
        a.eps = op.has_arg("Eps") ? (float)op.arg_float("Eps") : 1e-5f;
        a.scale = op.has_arg("Scale") ? (float)op.arg_float("Scale") : 1.0f;
        size_t ri = 1;
        if (a.op == RO_RMSNORM && op.reads.size() > ri && op.reads[ri].nelems() == a.cols) {
            a.weight_f32 = (op.reads[ri].dtype == DT_F32 && in.dtype != DT_F32) ? 1 : 0;
            if (!a.weight_f32 && op.reads[ri].dtype != in.dtype) throw Error(E_MODEL, "RMSNorm: the weight must have the rows' type or be FP32");
            a.weight = tensor_ptr(op.reads[ri++]);
        }
        if (op.has_arg("Residual") && op.arg_bool("Residual")) {
            if (op.reads.size() <= ri || op.results.size() < 2) throw Error(E_MODEL, op.type + ": residual form needs 2 results");
            a.residual = tensor_ptr(op.reads[ri]);
            a.res_out = tensor_ptr(op.results[1]);
        }
        if (a.op == RO_SOFTMAX && op.has_arg("Mask") && op.arg_bool("Mask")) {
            // additive mask [.., R, cols] broadcast over the leading dims: row r of the input uses mask row r % R
            if (op.reads.size() <= ri) throw Error(E_MODEL, "Softmax: mask tensor missing");
            const TensorDesc &mk = op.reads[ri++];
            auto ms = mk.shape4();
            auto mst = mk.strides4();
            if (mk.dtype != in.dtype || ms[3] != a.cols || ms[0] != 1 || ms[1] != 1 || sh[2] % ms[2] != 0 || (ms[2] != sh[2] && ms[2] != 1))
                throw Error(E_UNSUPPORTED, "Softmax: the mask must be [1, 1, rows or 1, cols] of the input's type");
            a.mask = tensor_ptr(mk);
            a.mask_ld = mst[3];
            a.mask_rows = (int32_t)ms[2];
        }
        const int V = (int)(16 / dtype_size(in.dtype));
        bool ok = (a.cols % V == 0) && aligned16(a.in) && aligned16(a.out) && (a.in_ld % V == 0) && (a.out_ld % V == 0);
        if (a.weight) ok = ok && aligned16(a.weight);
        if (a.mask) ok = ok && aligned16(a.mask) && (a.mask_ld % V == 0);
        if (a.residual) ok = ok && aligned16(a.residual) && aligned16(a.res_out);
        if (!ok) throw Error(E_UNSUPPORTED, op.type + ": rows must be 16-byte aligned and a multiple of 16 bytes long");
        if (!(in.dtype == DT_F32 || in.dtype == DT_F16 || in.dtype == DT_BF16)) throw Error(E_UNSUPPORTED, op.type + ": floating-point only");
        std::string part_note;
        if (tg && !full_range(tg->task_range, num_tasks(op))) {
            // a task is one row: the rows task_b, task_b + task_s, ... are a view with a larger row pitch
            if (num_tasks(op) != a.rows) throw Error(E_UNSUPPORTED, op.type + ": a partial TaskRange needs one task per row");
            const int64_t b = tg->task_range.b, st = std::max<int64_t>(1, tg->task_range.s), e = std::min<int64_t>(tg->task_range.e, a.rows);
            if (a.mask && a.mask_rows > 1 && (st != 1 || b % a.mask_rows))
                throw Error(E_UNSUPPORTED, "Softmax: a partial TaskRange must start on a mask period and have step 1");
            const size_t es = dtype_size(in.dtype);
            a.in = reinterpret_cast<const char *>(a.in) + (size_t)b * a.in_ld * es;
            a.out = reinterpret_cast<char *>(a.out) + (size_t)b * a.out_ld * es;
            if (a.residual) {
                a.residual = reinterpret_cast<const char *>(a.residual) + (size_t)b * a.in_ld * es;
                a.res_out = reinterpret_cast<char *>(a.res_out) + (size_t)b * a.in_ld * es;  // res_out rows follow the input's pitch
            }
            a.rows = e > b ? (e - b + st - 1) / st : 0;
            a.in_ld *= st;
            a.out_ld *= st;
            part_note = " tasks [" + std::to_string(b) + "," + std::to_string(e) + (st != 1 ? "," + std::to_string(st) : "") + ")";
        }
        // warps that share a row so that each lane keeps at most 8 16-byte vectors of it in registers
        {
            const int64_t nv = a.cols / V;
            int gw = 1;
            while (gw < 16 && nv > (int64_t)32 * gw * 8) gw *= 2;
            a.warps_per_row = nv <= (int64_t)32 * gw * 8 ? gw : 0;
        }
        // streaming through shared memory (bulk copies): rows of 1 KiB .. 48 KiB, enough rows
        // to give every warp several; 16 warps first, then up to 3 row buffers per warp, within 192 KiB
        {
            const int64_t row_bytes = a.cols * (int64_t)dtype_size(in.dtype);
            const int64_t buf = (row_bytes + 127) / 128 * 128;
            const char *e = getenv("ARKB_ROW_STAGED");
            const bool want = e ? atoi(e) != 0 : true;
            if (want && row_bytes >= 1024 && buf <= 96 * 1024 && a.rows >= 4 * proc.count()) {
                // all row buffers that fit are kept in flight; warps first (they do the arithmetic), then depth
                const int64_t wbytes = a.weight ? (a.cols * (a.weight_f32 ? 4 : (int64_t)dtype_size(in.dtype)) + 127) / 128 * 128 : 0;
                a.weight_smem = a.weight && wbytes <= 64 * 1024 ? 1 : 0;
                const int64_t total = (192 * 1024 - (a.weight_smem ? wbytes : 0)) / buf;
                a.staged_bufs = (int32_t)std::max<int64_t>(1, std::min<int64_t>(3, total / 16));
                a.staged_warps = (int32_t)std::min<int64_t>(16, total / a.staged_bufs);
            }
        }
        push(s, op.type + " " + op.name + " rows=" + std::to_string(a.rows) + " cols=" + std::to_string(a.cols) +
                    " warps/row=" + std::to_string(a.warps_per_row) +
                    (a.staged_warps ? " staged(" + std::to_string(a.staged_warps) + " warps x " + std::to_string(a.staged_bufs) + " rows)" : "") + part_note);
    }

    // ---- matmul --------------------------------------------------------------------
    struct MM {
        int64_t M, N, K;
        bool ta, tb;
        int64_t bc, bn;
    };

    static int act_code(const std::string &t) {
        if (t == "Relu") return ACT_RELU;
        if (t == "Gelu") return ACT_GELU;
        if (t == "Sigmoid") return ACT_SIGMOID;
        if (t == "Silu") return ACT_SILU;
        return -1;
    }

    // Number of ops of the plan (other than `except`) that read buffer `buf`.
    int other_readers(int64_t buf, const OpDesc *except) const {
        int n = 0;
        for (auto &ti : plan.task_infos)
            for (auto &op : ti.ops) {
                if (&op == except) continue;
                for (auto &t : op.reads)
                    if (t.buffer_id == buf) ++n;
            }
        return n;
    }

    // Operators of the same task folded into a weight-streaming matmul (SK_GEMV): a prologue applied to the
    // activations while they are staged, and a residual added to the result.
    struct GemvFuse {
        int pro = GP_NONE;
        const TensorDesc *x = nullptr;        // what the prologue reads (takes the place of the matmul's first operand)
        const TensorDesc *pro_a = nullptr;    // rmsnorm weight / second factor of the mul
        const TensorDesc *pro_b = nullptr;    // rmsnorm residual
        const TensorDesc *pro_out = nullptr;  // where x + residual is kept
        float eps = 1e-5f;
        const TensorDesc *residual = nullptr; // added to the matmul's result
        const TensorDesc *out = nullptr;      // result tensor of the last folded operator
        int push_ord = -1;                    // >= 0: ordinal of the one-shot all_reduce whose push this matmul does
    };
    std::vector<OpDesc> fused_ops;          // row operators that stand for a chain of the plan's operators
    std::map<size_t, size_t> chain_pgs;     // first processor group of such a chain -> index into fused_ops
    bool gemv_pushed = false;  // set by lower_matmul when the push of a one-shot all_reduce was folded in
    // Operators folded across processor groups in the decode chain:
    const OpDesc *rope_for_attention = nullptr;  // a Rope whose only reader is the DecodeAttention of the next group
    struct PendingMerge {                        // a DecodeAttention whose chunks the weight-streaming matmul of the next group merges
        int64_t buffer_id = -1;
        const float *ws = nullptr;
        size_t ws_bytes = 0;
        int chunks = 0, group = 0, kv_heads = 0;
        int64_t B = 0, Hq = 0;
    } pending_merge;
    size_t cur_pg = 0, pending_merge_pg = 0;
    // A one-shot all_reduce (with the Add that consumes it) whose sum stage was left out: the weight-streaming matmuls of
    // the processor groups that follow (RMSNorm folded in) add the slots up themselves; the first of them also stores
    // the sum (+ residual) for later readers.
    struct PendingSum {
        int64_t buffer_id = -1;     // buffer of the tensor the sum stage would have written
        int ord = 0;                // ordinal of the all_reduce + 1
        bool has_residual = false, stored = false;
        TensorDesc residual, out;   // the Add's other operand; the tensor to store
        int64_t rows = 0, cols = 0;
    } pending_sum;
    // processor group `k` is [RMSNorm(x), Matmul] that lower_task_group folds into one weight-streaming stage, x on `buffer`
    bool sum_consumer(size_t k, int64_t buffer, int64_t rows, int64_t cols) const {
        if (k >= plan.processor_groups.size()) return false;
        const ProcessorGroup &g = plan.processor_groups[k];
        if (g.resource_groups.size() != 1 || g.resource_groups[0].task_groups.size() != 1) return false;
        const TaskGroup &tg = g.resource_groups[0].task_groups[0];
        const TaskInfo &ti = plan.task(tg.task_id);
        if (ti.ops.size() < 2) return false;
        const OpDesc &n = ti.ops[0], &m = ti.ops[1];
        if (n.type != "RMSNorm" || m.type != "Matmul" || n.reads.empty() || n.results.empty() || m.reads.empty()) return false;
        if (n.has_arg("Residual") && n.arg_bool("Residual")) return false;
        const TensorDesc &x = n.reads[0], &mx = m.reads[0];
        if (x.buffer_id != buffer || !x.dense() || x.shape4()[2] != rows || x.shape4()[3] != cols || x.shape4()[0] * x.shape4()[1] != 1) return false;
        if (m.reads[0].id != n.results[0].id || other_readers(n.results[0].buffer_id, &m) != 0) return false;
        return matmul_is_gemv(m, tg) && x.shape4() == mx.shape4() && x.dtype == mx.dtype;
    }
    static bool fold_decode_chain() { const char *e = getenv("ARKB_FOLD_DECODE"); return e ? atoi(e) != 0 : true; }
    // Rope of the new token's query whose only reader is the DecodeAttention that opens the next processor group: the
    // attention rotates q while it loads it (no stage, no barrier for the rotation)
    bool rope_feeds_next_attention(const OpDesc &o) const {
        if (!fold_decode_chain() || o.type != "Rope" || o.reads.size() != 2 || o.results.empty()) return false;
        const OpDesc *nx = first_op_of(cur_pg + 1);
        return nx && nx->type == "DecodeAttention" && nx->reads.at(0).buffer_id == o.results[0].buffer_id &&
               o.results[0].buffer_id != o.reads[0].buffer_id && o.reads[0].dense() && o.results[0].dense() && nx->reads[0].dense() &&
               o.reads[0].dtype == nx->reads[0].dtype && o.reads[1].dtype == o.reads[0].dtype && o.reads[1].dense() &&
               o.reads[1].nelems() == 128 && o.reads[0].shape4()[3] == 128 && o.reads[0].nelems() == nx->reads[0].nelems() &&
               other_readers(o.results[0].buffer_id, nx) == 0;
    }
    // first operator that does something of processor group `k` (null when the group is not a plain single-task group)
    const OpDesc *first_op_of(size_t k, const TaskGroup **tg_out = nullptr) const {
        if (k >= plan.processor_groups.size()) return nullptr;
        const ProcessorGroup &g = plan.processor_groups[k];
        if (g.resource_groups.size() != 1 || g.resource_groups[0].task_groups.size() != 1) return nullptr;
        const TaskGroup &tg = g.resource_groups[0].task_groups[0];
        for (auto &o : plan.task(tg.task_id).ops) {
            if (o.is_virtual || o.type == "Reshape" || o.type == "Identity" || o.type == "Refer" || o.type == "Noop") continue;
            if (tg_out) *tg_out = &tg;
            return &o;
        }
        return nullptr;
    }

    // an AllReduce the engine runs one-shot (every rank pushes its tensor into every rank's staging slots)
    bool all_reduce_is_one_shot(const OpDesc &op) const {
        if (op.type != "AllReduce" || op.results.empty() || env.nranks < 2) return false;
        const TensorDesc &t = op.results[0];
        const size_t bytes = (size_t)t.nelems() * dtype_size(t.dtype);
        const std::string algo = op.config.is_object() && op.config.contains("Algo") ? op.config.at("Algo").as_string() : "auto";
        return t.dense() && ((algo == "oneshot") || (algo == "auto" && bytes <= 256 * 1024)) && bytes <= lay.comm_stage_bytes / kMaxPeers;
    }

    // ops[j] is a one-shot AllReduce and ops[j+1] the Add of its sum with a dense tensor of the same shape: the Add
    const OpDesc *add_after_all_reduce(const TaskInfo &ti, size_t j) const {
        if (j + 1 >= ti.ops.size() || !all_reduce_is_one_shot(ti.ops[j])) return nullptr;
        const OpDesc &ar = ti.ops[j], &nx = ti.ops[j + 1];
        if (nx.type != "Add" || nx.reads.size() != 2 || nx.results.empty()) return nullptr;
        const TensorDesc &t = ar.results[0];
        const bool first = nx.reads[0].id == t.id, second = nx.reads[1].id == t.id;
        if (first == second) return nullptr;
        const TensorDesc &other = first ? nx.reads[1] : nx.reads[0];
        if (!other.dense() || !nx.results[0].dense() || other.shape4() != t.shape4() || nx.results[0].shape4() != t.shape4() ||
            other.dtype != t.dtype || nx.results[0].dtype != t.dtype)
            return nullptr;
        for (auto &tk : plan.task_infos)  // the bare sum must not be used elsewhere
            for (auto &o : tk.ops) {
                if (&o == &nx || &o == &ar) continue;
                for (auto &rd : o.reads)
                    if (rd.buffer_id == t.buffer_id) return nullptr;
            }
        return &nx;
    }

    static bool gemv_wanted() {
        const char *e = getenv("ARKB_GEMV");
        return e ? atoi(e) != 0 : true;
    }
    // shapes the weight-streaming stage takes (the same test decides inside lower_matmul)
    static bool gemv_shape_ok(bool full, bool ta, bool tb, int64_t M, int64_t N, int64_t K, int64_t batches, int64_t lda) {
        return full && !ta && M <= kGemvMaxM && batches == 1 && K % 8 == 0 &&
               (tb ? K >= 512 : N % 8 == 0 && N >= 256 && M * K * 2 <= 160 * 1024) && lda % 8 == 0 && N * K >= 65536;
    }
    bool matmul_is_gemv(const OpDesc &op, const TaskGroup &tg) const {
        if (op.type != "Matmul" || op.reads.size() < 2 || op.results.empty()) return false;
        const TensorDesc &A = op.reads[0], &B = op.reads[1], &C = op.results[0];
        if (A.dtype != B.dtype || (A.dtype != DT_F16 && A.dtype != DT_BF16)) return false;
        const bool ta = op.arg_bool("TransposeInput");
        const bool tb = B.shape.size() == 1 ? true : op.arg_bool("TransposeOther");
        auto ash = A.shape4(), bsh = B.shape4(), csh = C.shape4();
        int64_t M = A.shape.size() == 1 ? 1 : ash[2], K = ash[3];
        if (ta) std::swap(M, K);
        int64_t N = bsh[3];
        if (tb) N = bsh[2];
        const size_t es = dtype_size(A.dtype);
        auto ast = A.strides4(), bst = B.strides4();
        const bool aligned = aligned16(tensor_ptr(A)) && aligned16(tensor_ptr(B)) && (ast[3] * es) % 16 == 0 && (bst[3] * es) % 16 == 0;
        return gemv_wanted() && aligned && env.encode_tmap &&
               gemv_shape_ok(full_range(tg.task_range, num_tasks(op)), ta, tb, M, N, K, csh[0] * csh[1], ast[3]);
    }

    // A tensor-core matmul (the ordinary tiled form: more than 128 rows, operands the tensor maps can describe, the
    // whole task range) whose epilogue can combine the accumulator with a tensor of the result's layout.
    bool matmul_takes_epilogue_operand(const OpDesc &op, const TaskGroup &tg, const TensorDesc &other, const TensorDesc &out) const {
        if (op.type != "Matmul" || op.reads.size() < 2 || op.results.empty() || !env.encode_tmap) return false;
        const TensorDesc &A = op.reads[0], &B = op.reads[1], &C = op.results[0];
        if (A.dtype != B.dtype || A.dtype != C.dtype || (A.dtype != DT_F16 && A.dtype != DT_BF16)) return false;
        if (other.dtype != C.dtype || out.dtype != C.dtype || other.shape4() != C.shape4() || out.shape4() != C.shape4() ||
            other.strides4() != out.strides4())
            return false;
        if (!full_range(tg.task_range, num_tasks(op)) || matmul_is_gemv(op, tg)) return false;
        const bool ta = op.arg_bool("TransposeInput");
        auto ash = A.shape4(), ast = A.strides4(), bst = B.strides4();
        const int64_t M = ta ? ash[3] : (A.shape.size() == 1 ? 1 : ash[2]);
        if (M <= 128) return false;  // those may run in the swapped / split-K forms
        const size_t es = 2;
        return aligned16(tensor_ptr(A)) && aligned16(tensor_ptr(B)) && aligned16(tensor_ptr(other)) && (ast[3] * es) % 16 == 0 &&
               (bst[3] * es) % 16 == 0 && (ast[2] * ast[3] * es) % 16 == 0 && (bst[2] * bst[3] * es) % 16 == 0;
    }

    void lower_matmul(const OpDesc &op, const Range &proc, const TaskGroup &tg, int act, const TensorDesc *act_out,
                      const OpDesc *fuse_ar = nullptr, const GemvFuse *gf = nullptr, const TensorDesc *epi = nullptr,
                      int epi_mode = 0 /* 0: add, 1: multiply, 2: rotary table [rope_rows][rope_cols] */, int64_t rope_rows = 0,
                      int64_t rope_cols = 0) {
        const TensorDesc &A = op.reads.at(0), &B = op.reads.at(1);
        const TensorDesc &C = act_out ? *act_out : op.results.at(0);
        const bool ta = op.arg_bool("TransposeInput");
        // a 1-D `other` is a column vector [K]: the same memory as a K-major [1, K] matrix
        const bool tb = B.shape.size() == 1 ? true : op.arg_bool("TransposeOther");
        if (A.dtype != B.dtype || A.dtype != C.dtype) throw Error(E_MODEL, "Matmul: operand data types differ");
        auto ash = A.shape4(), bsh = B.shape4(), csh = C.shape4();
        auto ast = A.strides4(), bst = B.strides4(), cst = C.strides4();
        // problem size (ark/ops/ops_matmul.cpp:13-42)
        int64_t M = A.shape.size() == 1 ? 1 : ash[2], K = ash[3];
        if (ta) std::swap(M, K);
        int64_t N = bsh[3], K2 = bsh[2];
        if (tb) std::swap(N, K2);
        if (K != K2) throw Error(E_MODEL, "Matmul: inner dimensions mismatch");
        if (csh[2] != M || csh[3] != N) throw Error(E_MODEL, "Matmul: output shape mismatch");
        const int64_t bn = csh[0], bc = csh[1];
        for (int d = 0; d < 2; ++d) {
            if ((ash[d] != 1 && ash[d] != csh[d]) || (bsh[d] != 1 && bsh[d] != csh[d]))
                throw Error(E_MODEL, "Matmul: batch dimensions do not broadcast");
        }
        const size_t es = dtype_size(A.dtype);
        const int64_t lda = ast[3], ldb = bst[3], ldc = cst[3];
        char *pa = tensor_ptr(A), *pb = tensor_ptr(B), *pc = tensor_ptr(C);
        const bool tma_ok = (A.dtype == DT_F16 || A.dtype == DT_BF16) && aligned16(pa) && aligned16(pb) &&
                            (lda * es) % 16 == 0 && (ldb * es) % 16 == 0 && (ast[2] * lda * es) % 16 == 0 &&
                            (bst[2] * ldb * es) % 16 == 0 && env.encode_tmap;
        const int64_t ntasks = num_tasks(op);
        const bool full = full_range(tg.task_range, ntasks);
        if (!tma_ok) {
            if (!full) throw Error(E_UNSUPPORTED, "Matmul: partial TaskRange needs 16-byte aligned fp16/bf16 operands");
            if (epi) throw Error(E_INTERNAL, "Matmul: epilogue operand on the CUDA-core form");
            Stage s = new_stage(SK_GEMM_SIMT, proc);
            GemmSimtArgs &g = s.gs;
            acc_begin();
            rd(A); rd_streamed(B); wr(C);
            g.A = pa; g.B = pb; g.C = pc;
            g.lda = lda; g.ldb = ldb; g.ldc = ldc;
            g.a_stride_c = ash[1] > 1 ? ast[2] * ast[3] : 0;
            g.a_stride_n = ash[0] > 1 ? ast[1] * ast[2] * ast[3] : 0;
            g.b_stride_c = bsh[1] > 1 ? bst[2] * bst[3] : 0;
            g.b_stride_n = bsh[0] > 1 ? bst[1] * bst[2] * bst[3] : 0;
            g.c_stride_c = cst[2] * cst[3];
            g.c_stride_n = cst[1] * cst[2] * cst[3];
            g.M = (int32_t)M; g.N = (int32_t)N; g.K = (int32_t)K;
            g.batch_c = (int32_t)bc; g.batch_n = (int32_t)bn;
            g.trans_a = ta; g.trans_b = tb;
            g.dtype = A.dtype; g.act = act;
            push(s, "Matmul(simt) " + op.name + " M=" + std::to_string(M) + " N=" + std::to_string(N) + " K=" + std::to_string(K));
            return;
        }
        // One or two rows of activations against an unbatched weight matrix: the work is a read of the weights at
        // HBM speed; it runs on the CUDA cores with the activations in shared memory. (From three rows on the
        // multiply-adds outweigh the read and the swapped tensor-core form below is faster.)
        {
            const int64_t P = proc.count();
            const bool shapes_ok = gemv_shape_ok(full, ta, tb, M, N, K, bn * bc, lda);
            if (gf && !(gemv_wanted() && shapes_ok)) throw Error(E_INTERNAL, "operators were folded into a matmul that is not weight-streaming");
            if (gemv_wanted() && shapes_ok) {
                Stage s = new_stage(SK_GEMV, proc);
                GemvArgs &g = s.gv;
                g.out = pc; g.x = pa; g.w = pb;
                const bool merge_here = pending_merge.buffer_id >= 0 && pending_merge.buffer_id == A.buffer_id;
                if (merge_here) {
                    if ((gf && gf->pro != GP_NONE) || M != pending_merge.B || K != pending_merge.Hq * 128 || !A.dense())
                        throw Error(E_INTERNAL, "decode attention merge folded into a matmul that cannot take it");
                    g.pro = GP_ATTN_MERGE;
                    g.pro_a = pending_merge.ws;
                    g.mg_chunks = pending_merge.chunks; g.mg_group = pending_merge.group; g.mg_kv_heads = pending_merge.kv_heads;
                }
                const bool sum_here = gf && gf->pro == GP_RMSNORM && gf->x && pending_sum.buffer_id >= 0 &&
                                      gf->x->buffer_id == pending_sum.buffer_id && !merge_here;
                if (sum_here && (gf->pro_b || M != pending_sum.rows || K != pending_sum.cols))
                    throw Error(E_INTERNAL, "one-shot all_reduce sum folded into a matmul that cannot take it");
                if (gf) {
                    // the prologue's input stands in for the first operand; every folded operand shares its row pitch
                    auto same_rows = [&](const TensorDesc *t) { return !t || (t->strides4()[3] == gf->x->strides4()[3] && aligned16(tensor_ptr(*t))); };
                    if (gf->x) {
                        if (gf->x->strides4()[3] != lda || lda % 8 || !aligned16(tensor_ptr(*gf->x)) || !same_rows(gf->pro_b) || !same_rows(gf->pro_out) ||
                            (gf->pro == GP_MUL && !same_rows(gf->pro_a)))
                            throw Error(E_UNSUPPORTED, "folded operands of a weight-streaming matmul must share one 16-byte aligned row pitch");
                        g.x = tensor_ptr(*gf->x);
                    }
                    if (!merge_here) g.pro = gf->pro;
                    if (!merge_here) g.pro_a = gf->pro_a ? tensor_ptr(*gf->pro_a) : nullptr;
                    g.pro_b = gf->pro_b ? tensor_ptr(*gf->pro_b) : nullptr;
                    g.pro_out = gf->pro_out ? tensor_ptr(*gf->pro_out) : nullptr;
                    g.pro_eps = gf->eps;
                    if (sum_here) {
                        g.src_ord = pending_sum.ord;
                        if (pending_sum.has_residual) g.pro_b = tensor_ptr(pending_sum.residual);
                        if (!pending_sum.stored) g.pro_out = tensor_ptr(pending_sum.out);
                        if ((g.pro_b && !aligned16(g.pro_b)) || (g.pro_out && !aligned16(g.pro_out)))
                            throw Error(E_UNSUPPORTED, "AllReduce folded into a weight-streaming matmul: operands must be 16-byte aligned");
                    }
                    if (gf->residual) {
                        if (gf->residual->strides4()[3] != ldc) throw Error(E_UNSUPPORTED, "residual of a weight-streaming matmul must have the result's row pitch");
                        g.residual = tensor_ptr(*gf->residual);
                    }
                }
                g.ldx = lda; g.ldw = ldb; g.ldo = ldc;
                g.M = (int32_t)M; g.N = (int32_t)N; g.K = (int32_t)K;
                g.w_is_nk = tb ? 1 : 0;
                g.dtype = A.dtype;
                g.act = act < 0 ? ACT_NONE : act;
                if (tb) {
                    // CTAs = k-ranges x row blocks; a warp walks whole groups of RW rows, so the time of the stage is
                    // (groups per warp, rounded up) x (steps per group). Pick the rows per group and the number of
                    // k-ranges with the least such time: fewer rows per group when there are not enough rows to go
                    // round (the activations are then re-read from shared memory more often), more than one k-range
                    // only when it pays for the barrier and the pass over the partials it adds.
                    // small matrices (per CTA at most 384 KiB of weights) take the light walker: half the loads per step
                    bool light = (int64_t)N * K * (int64_t)es <= P * (384ll << 10);
                    if (const char *e = getenv("ARKB_GEMV_LIGHT")) light = atoi(e) != 0;
                    g.light = light ? 1 : 0;
                    const int64_t warps = kThreads / 32, loads = (M == 1 ? 8 : 4) / (light ? 2 : 1);  // 16-byte loads per lane and step
                    auto kper_of = [&](int64_t sp) { return ((K + sp - 1) / sp + 255) / 256 * 256; };
                    const double step_us = 256.0 * loads * es * (double)(P * warps) / 6.5e6;
                    int64_t splits = 0, best_rw = loads;
                    double best = 1e30;
                    for (int64_t RW = loads; RW >= 1; RW /= 2) {
                        const int64_t VC = loads / RW;
                        for (int64_t sp = 1; sp <= std::min<int64_t>(P, 32); ++sp) {
                            const int64_t kp = kper_of(sp), eff = (K + kp - 1) / kp;
                            if (eff != sp) continue;
                            if (M * kp * 4 > 160 * 1024) continue;
                            if (kp < 1024 && sp > 1) break;
                            const int64_t cps = P / eff;
                            const int64_t rows_cta = (N + cps - 1) / cps;
                            const int64_t rounds = ((rows_cta + RW - 1) / RW + warps - 1) / warps;
                            const double steps = (double)((kp + 256 * VC - 1) / (256 * VC));
                            const double t = (double)rounds * (steps + 1.5) * step_us * (1.0 + 0.03 * (double)(VC - 1)) +
                                             (eff > 1 ? 7.0 : 0.0);
                            if (t < best - 1e-9) { best = t; splits = eff; best_rw = RW; }
                        }
                    }
                    g.rows_together = (int32_t)best_rw;
                    const int64_t kper = kper_of(splits);
                    g.kper = (int32_t)kper;
                    g.splits = (int32_t)splits;
                    g.ctas_per_split = (int32_t)(P / splits);
                } else {
                    // items = column blocks x k-ranges, one warp each, dealt round-robin over all warps: enough
                    // k-ranges to give every warp an item, and the count whose last wave is fullest
                    const int64_t nblocks = (N + 255) / 256, W = P * (kThreads / 32);
                    int64_t best_sp = 1;
                    double best = -1;
                    for (int64_t sp = 1; sp <= 256; ++sp) {
                        const int64_t kper = (K + sp - 1) / sp;
                        if (kper < 64 && sp > 1) break;
                        const int64_t items = nblocks * ((K + kper - 1) / kper);
                        const double eff = (double)items / (double)(((items + W - 1) / W) * W);
                        if (eff > best + 0.03) { best = eff; best_sp = sp; }
                    }
                    const int64_t kper = (K + best_sp - 1) / best_sp;
                    g.kper = (int32_t)kper;
                    g.splits = (int32_t)((K + kper - 1) / kper);
                    g.nblocks = (int32_t)nblocks;
                }
                if (g.splits > 1) {
                    if (!env.workspace) {
                        g.splits = 1;  // no scratch in this pass (plan checks): shape of the stage list is all that matters
                    } else {
                        const size_t bytes = (size_t)g.splits * M * N * sizeof(float);
                        g.ws = reinterpret_cast<float *>(env.workspace + prog.workspace_bytes);
                        prog.workspace_bytes += (bytes + 255) / 256 * 256;
                    }
                }
                const int act_final = g.act;
                if (g.splits > 1) g.act = ACT_NONE;
                if (g.residual && act_final != ACT_NONE) throw Error(E_INTERNAL, "residual and activation folded into one matmul");
                gemv_pushed = false;
                if (gf && gf->push_ord >= 0 && g.splits == 1 && ldc == N) {
                    g.push_ord = gf->push_ord + 1;
                    g.push_stage_bytes = lay.comm_stage_bytes;
                    gemv_pushed = true;
                }
                const GemvArgs gv = g;
                acc_begin();
                if (merge_here) {
                    rd_raw(pending_merge.ws, pending_merge.ws_bytes);
                    pending_merge = PendingMerge();
                } else {
                    rd(A);
                }
                if (sum_here) {
                    if (pending_sum.has_residual) rd(pending_sum.residual);
                    if (!pending_sum.stored) wr(pending_sum.out);
                    pending_sum.stored = true;
                }
                rd_streamed(B);
                if (gf) {
                    for (const TensorDesc *t : {sum_here ? nullptr : gf->x, gf->pro_a, gf->pro_b, gf->residual})  // a folded sum is read from the staging slots, not from x
                        if (t) rd(*t);
                    if (gf->pro_out) wr(*gf->pro_out);
                }
                if (gv.splits > 1) wr_raw(gv.ws, (size_t)gv.splits * M * N * sizeof(float));
                else wr(C);
                if (gv.push_ord) acc.opaque = true;  // also stores into every rank's all_reduce slots
                push(s, std::string("Matmul(gemv) ") + op.name + " M=" + std::to_string(M) + " N=" + std::to_string(N) + " K=" +
                            std::to_string(K) + (tb ? " W:[N,K]" : " W:[K,N]") + " k-ranges=" + std::to_string(gv.splits) + " x " +
                            std::to_string(gv.kper) + (tb ? " ctas/range=" + std::to_string(gv.ctas_per_split) + " rows/warp-step=" + std::to_string(gv.rows_together) + (gv.light ? " light" : "") : "") +
                            (gv.src_ord ? (gv.pro_b ? " <-all_reduce sum +residual" : " <-all_reduce sum") : "") +
                            (gv.pro == GP_RMSNORM ? " <-rmsnorm" : gv.pro == GP_MUL ? " <-mul" : gv.pro == GP_ATTN_MERGE ? " <-attention merge" : "") + (gv.residual ? " +residual" : "") +
                            (gv.push_ord ? " ->all_reduce slots" : "") +
                            (gv.act ? " act=" + std::to_string(gv.act) : ""));
                if (gv.splits > 1) {
                    emit_sync(proc);
                    Stage r = new_stage(SK_SPLITK_REDUCE, proc);
                    SplitKReduceArgs &a = r.sr;
                    a.C = pc;
                    a.bias = gv.residual;  // a folded residual is added by the sum stage
                    a.ws = gv.ws;
                    a.ldc = ldc;
                    a.c_stride_c = cst[2] * cst[3];
                    a.c_stride_n = cst[1] * cst[2] * cst[3];
                    a.M = (int32_t)M; a.N = (int32_t)N;
                    a.batch_c = 1; a.batch_n = 1;
                    a.splits = gv.splits;
                    a.dtype = A.dtype;
                    a.act = act_final;
                    acc_begin();
                    rd_raw(gv.ws, (size_t)gv.splits * M * N * sizeof(float));
                    if (gf && gf->residual) rd(*gf->residual);
                    wr(C);
                    push(r, "  split-K sum " + op.name + " splits=" + std::to_string(a.splits));
                }
                return;
            }
        }
        // Skinny problems (few rows of activations against a large weight matrix, the
        // decode case) are run swapped: the weights become the 128-row A operand that fills
        // the shared-memory ring, the activations the narrow B operand.
        // up to 128 rows too when the ordinary form could not spread over half of the CTAs (few, long tiles: the split-K
        // of the swapped form then puts every SM to work on the weights)
        bool swapped = full && !ta && M <= 64;
        if (full && !ta && !swapped && M <= 128 && !fuse_ar) {
            const int64_t Pq = prog.pair_mode ? proc.count() / 2 : proc.count();
            const int64_t min_n = tb ? (prog.pair_mode ? 32 : 16) : (prog.pair_mode ? 128 : 64);
            const int64_t units = bn * bc * ((N + min_n - 1) / min_n);
            int factor = 3;
            if (const char *e = getenv("ARKB_SWAP128_FACTOR")) factor = atoi(e);
            swapped = units * factor < Pq;
        }
        if (epi && swapped) throw Error(E_INTERNAL, "Matmul: epilogue operand on the swapped form");
        Stage s = new_stage(SK_GEMM, proc);
        GemmArgs &g = s.gm;
        g.C = pc;
        g.bias = epi ? tensor_ptr(*epi) : nullptr;
        g.bias_mul = epi ? epi_mode : 0;
        g.rope_rows = (int32_t)rope_rows; g.rope_cols = (int32_t)rope_cols;
        g.ldc = ldc;
        g.c_stride_c = cst[2] * cst[3];
        g.c_stride_n = cst[1] * cst[2] * cst[3];
        g.M = (int32_t)M; g.N = (int32_t)N; g.K = (int32_t)K;
        g.batch_c = (int32_t)bc; g.batch_n = (int32_t)bn;
        g.a_bc = ash[1] > 1; g.a_bn = ash[0] > 1; g.b_bc = bsh[1] > 1; g.b_bn = bsh[0] > 1;
        g.a_mn_major = ta ? 1 : 0;   // A stored [K, M]: M is the inner dim
        g.b_mn_major = tb ? 0 : 1;   // B stored [K, N]: N is the inner dim
        if (swapped) {
            std::swap(g.M, g.N);
            std::swap(g.a_bc, g.b_bc);
            std::swap(g.a_bn, g.b_bn);
            g.a_mn_major = tb ? 0 : 1;  // the weights in the A role
            g.b_mn_major = 0;           // the activations [M, K] in the B role
            g.out_transposed = 1;
        }
        g.dtype = A.dtype;
        g.act = act < 0 ? ACT_NONE : act;
        g.c_vec = (aligned16(pc) && ldc % 8 == 0 && g.c_stride_c % 8 == 0 && g.c_stride_n % 8 == 0) ? 1 : 0;
        const int tile_m = prog.pair_mode ? 256 : 128;
        g.tile_m = tile_m;
        const int64_t P = prog.pair_mode ? proc.count() / 2 : proc.count();
        const int64_t tiles_m = ((swapped ? N : M) + tile_m - 1) / tile_m;
        if (swapped) {
            g.tile_n = (int32_t)((M + 15) / 16 * 16);
            g.plan_tiles = 0;
            g.tiles_m = (int32_t)tiles_m;
            g.tiles_n = 1;
            g.raster_group = (int32_t)tiles_m;
            g.n_units = (int32_t)(bn * bc * tiles_m);
            // One bulk tensor copy per operand brings `kgroup` k-blocks into a ring slot: a producer thread that
            // issues one 16 KiB copy at a time tops out near 5.2 TB/s over all SMs, 32 KiB copies reach 6.3.
            // Needs whole k-blocks (K % 64 == 0) and at least 4 slots in shared memory.
            {
                const int64_t b_rows_k = prog.pair_mode ? g.tile_n / 2 : g.tile_n;
                const int64_t per_block = 16 * 1024 + b_rows_k * 128;
                int G = 1;
                if (K % 64 == 0) {
                    if (kSwappedRingBytes / (2 * per_block) >= 4) G = 2;
                }
                if (const char *e = getenv("ARKB_KGROUP")) G = std::max(1, std::min(G, atoi(e)));
                g.kgroup = G;
            }
            // Split K when the tiles alone cannot keep every CTA (pair) streaming weights: pick the
            // split with the least makespan in k-blocks. Partials go to scratch and a second stage
            // sums them in a fixed order (deterministic).
            const int64_t kblocks = (K + 63) / 64, tiles = g.n_units;
            int best_s = 1;
            int64_t best_kper = kblocks;
            double best = 1e30;
            for (int sp = 1; sp <= 32 && sp * 2 <= kblocks; ++sp) {
                const int64_t kper = ((kblocks + sp - 1) / sp + g.kgroup - 1) / g.kgroup * g.kgroup;
                const int64_t eff = (kblocks + kper - 1) / kper;
                const int64_t waves = (tiles * eff + P - 1) / P;
                const double cost = (double)waves * kper + 0.5 * eff;
                if (cost < best - 1e-9) { best = cost; best_s = (int)eff; best_kper = kper; }
            }
            if (best_s > 1 && env.workspace) g.kper = (int32_t)best_kper;
            if (best_s > 1 && env.workspace) {
                g.splits = best_s;
                g.n_units = (int32_t)(tiles * best_s);
                const size_t bytes = (size_t)best_s * bn * bc * M * N * sizeof(float);
                g.ws = reinterpret_cast<float *>(env.workspace + prog.workspace_bytes);
                prog.workspace_bytes += (bytes + 255) / 256 * 256;
            }
        } else if (full) {
            // tile_n: with many waves of tiles the widest tile is the most efficient; with few,
            // pick the width whose makespan (waves x tile width, plus a fixed cost per tile) is least,
            // so that skinny and small problems spread evenly over the CTAs.
            // a CTA stages whole 64-column chunks of a row-major (MN-major) B, so its share stays a multiple of 64
            // (a matmul fused with the all_reduce behind it stores its tiles as 32-column blocks)
            const int step = g.b_mn_major ? (prog.pair_mode ? 128 : 64) : (prog.pair_mode || fuse_ar ? 32 : 16);
            const int min_n = step;
            int tile_n = 256;
            int64_t want_splits = 1;
            // tall tiles (one CTA per tile only; off unless ARKB_TALL=1, 2 = wherever they are possible): 256 x tile_n per
            // CTA as two 128-row halves that share every B block, a third fewer operand bytes per flop at width 256.
            // Measured on the 7B prefill shapes they gain nothing: a k-block of a half still takes 0.53 us (the ring holds
            // 3 slots of 62 KiB instead of 4 of 46, so fewer bytes are in flight: the main loop follows the bytes in flight
            // over the load latency, not the bytes loaded), and both accumulator buffers belong to one tile, so the
            // epilogue (~5 us per half with direct stores) no longer overlaps the next tile: 2048 x 11008 x 4096 went from
            // 195 to 265 us, 2048 x 4096 x 11008 from 157 to 149, the layer from 0.91 to 1.02 ms.
            const char *tall_env = getenv("ARKB_TALL");
            const bool tall_on = tall_env && atoi(tall_env) != 0;
            const bool tall_forced = tall_env && atoi(tall_env) == 2;
            const bool may_tall = tall_on && !prog.pair_mode && M > 128 && !fuse_ar;  // not combined with the fused all_reduce (never run together)
            bool want_tall = false;
            {
                // Time model of a tile (microseconds), fitted to measurements of 2048 x 4096 x 4096 at every width: a
                // k-block takes the longest of its MMAs (0.4 us at width 256), of its operand loads (the CTA's A rows
                // plus its share of B, at ~90 GB/s per SM; CTA pairs were measured 1.35x slower per byte) and of a
                // floor of ~0.42 us that no tile width went below; a tile ~2 us more (pipeline fill, epilogue tail).
                // Few, long tiles (a narrow output with a long K: one rank's K/V projection) may also cut K into
                // ranges: fp32 partials go to scratch and a sum stage follows (~12 us for the barrier and the second stage, plus
                // the partials read back at ~4 TB/s). Rounds x tile time picks width and ranges together.
                const int64_t units256 = bn * bc * tiles_m * ((N + 255) / 256);
                static const bool old_model = []() { const char *e = getenv("ARKB_TILE_MODEL"); return e && atoi(e) == 0; }();
                static const bool splitk_on = []() { const char *e = getenv("ARKB_SPLITK_TILES"); return e ? atoi(e) != 0 : true; }();
                const bool may_split = splitk_on && env.workspace && !fuse_ar && !(epi && epi_mode != 0) && (N % 4) == 0 && !old_model;
                const int64_t kblocks = (K + 63) / 64;
                double best = 1e30;
                if (units256 < 8 * P) {
                    for (int c = 256; c >= min_n; c -= step) {
                        const int64_t units = bn * bc * tiles_m * ((N + c - 1) / c);
                        const double load = prog.pair_mode ? 1.35 * 1.42e-3 * (128 + c / 2.0) : 1.42e-3 * (128 + c);
                        const double tk = std::max(std::max(0.4 * c / 256.0, load), old_model ? 0.0 : 0.42);
                        for (int64_t sp = 1; sp <= (may_split ? 16 : 1); ++sp) {
                            if (sp > 1 && (units * sp > P || kblocks / sp < 8)) break;
                            const int64_t kp = (kblocks + sp - 1) / sp;
                            const int64_t waves = (units * sp + P - 1) / P;
                            double cost = old_model ? (double)waves * (c + 24) : (double)waves * ((double)kp * tk + 1.0 + 2.0 * c / 256.0);  // + fill, epilogue
                            if (sp > 1) cost += 12.0 + (double)sp * bn * bc * M * N * 4.0 / 4.0e6;  // measured: 2048 x 512 x 4096 gains nothing from 3 ranges
                            if (cost < best * (sp > 1 ? 0.9 : 1.0) - 1e-9) { best = cost; tile_n = c; want_splits = sp; }
                        }
                    }
                } else {
                    // many rounds: the widest tile (what the default above is); its cost, for the comparison with tall tiles
                    const int64_t units = bn * bc * tiles_m * ((N + 255) / 256);
                    const double load = prog.pair_mode ? 1.35 * 1.42e-3 * 256.0 : 1.42e-3 * 384.0;
                    best = (double)((units + P - 1) / P) * ((double)kblocks * std::max(0.4, load) + 3.0);
                }
                if (may_tall && !old_model) {
                    const int64_t tiles_m2 = (M + 255) / 256;
                    double best_tall = 1e30;
                    int tall_n = 256;
                    for (int c = 256; c >= std::max(min_n, 64); c -= step) {
                        const int64_t units = bn * bc * tiles_m2 * ((N + c - 1) / c);
                        const double tk = std::max(std::max(0.8 * c / 256.0, 1.42e-3 * (256 + c)), 0.5);
                        const int64_t waves = (units + P - 1) / P;
                        const double cost = (double)waves * ((double)kblocks * tk + 2.0 + 4.0 * c / 256.0);  // fill, two half-tile epilogues
                        if (cost < best_tall - 1e-9) { best_tall = cost; tall_n = c; }
                    }
                    if (best_tall < best * 0.95 || tall_forced) { want_tall = true; tile_n = tall_n; want_splits = 1; }
                }
            }
            if (const char *e = getenv("ARKB_TILE_N")) {  // experiments: force the tile width (rounded to what the mode allows)
                const int want = atoi(e);
                if (want >= min_n && want <= 256) tile_n = want / step * step;
            }
            if (N < tile_n) tile_n = (int)((N + step - 1) / step * step);  // narrow outputs: one tile covers N
            g.tile_n = tile_n;
            g.plan_tiles = 0;
            if (want_tall) {
                g.tall = 1;
                g.tile_m = 256;
            }
            const int64_t tiles_m = (M + g.tile_m - 1) / g.tile_m;
            g.tiles_m = (int32_t)tiles_m;
            g.tiles_n = (int32_t)((N + tile_n - 1) / tile_n);
            g.raster_group = (int32_t)std::min<int64_t>(tiles_m, 16);  // ~sqrt(#CTAs * tile_n / tile_m): least A+B bytes per wave
            g.n_units = (int32_t)(bn * bc * tiles_m * g.tiles_n);
            if (want_splits > 1) {
                const int64_t kblocks = (K + 63) / 64, units = g.n_units;
                const int64_t kp = (kblocks + want_splits - 1) / want_splits;
                const int64_t eff = (kblocks + kp - 1) / kp;
                if (eff > 1) {
                    g.splits = (int32_t)eff;
                    g.kper = (int32_t)kp;
                    g.n_units = (int32_t)(units * eff);
                    const size_t bytes = (size_t)eff * bn * bc * M * N * sizeof(float);
                    g.ws = reinterpret_cast<float *>(env.workspace + prog.workspace_bytes);
                    prog.workspace_bytes += (bytes + 255) / 256 * 256;
                }
            }
        } else {
            // honour the plan's task ids: tile id -> (n, c, tile_h, tile_w), w fastest
            auto tile = op.config.at("TileShapeMNK").as_int_vec();
            if (tile.size() != 3) throw Error(E_PLAN, "TileShapeMNK should have 3 elements");
            const int64_t ptm = tile[0], ptn = tile[1];
            if (ptm <= 0 || ptn <= 0) throw Error(E_PLAN, "TileShapeMNK must be positive");
            int tile_n = 0;
            for (int c = 256; c >= 16; c -= 16)
                if (ptn % c == 0 && (!prog.pair_mode || c % 32 == 0)) { tile_n = c; break; }
            if (!tile_n) throw Error(E_UNSUPPORTED, "Matmul: tile N of a partial TaskRange must be a multiple of 16");
            g.tile_n = tile_n;
            g.plan_tiles = 1;
            g.ptm = (int32_t)ptm; g.ptn = (int32_t)ptn;
            auto pad = C.padded.size() >= 2 ? C.padded : C.shape;
            const int64_t pM = pad[pad.size() - 2], pN = pad[pad.size() - 1];
            g.p_tiles_h = (int32_t)((pM + ptm - 1) / ptm);
            g.p_tiles_w = (int32_t)((pN + ptn - 1) / ptn);
            g.sub_m = (int32_t)((ptm + tile_m - 1) / tile_m);
            g.sub_n = (int32_t)(ptn / tile_n);
            g.task_b = (int32_t)tg.task_range.b;
            g.task_s = (int32_t)tg.task_range.s;
            g.n_units = (int32_t)(tg.task_range.count() * g.sub_m * g.sub_n);
        }
        // tensor maps: dims {inner, rows, C, N}
        // group > 1 (K-major operands only): the K axis is cut into 64-element blocks that become a dimension
        // of their own, {64, rows, K/64, C, N}, so that one box {64, rows, group} covers `group` k-blocks
        auto mk = [&](const TensorDesc &T, const std::vector<int64_t> &sh, const std::vector<int64_t> &st, char *base,
                      uint32_t box_inner, uint32_t box_rows, CUtensorMap *out, int swizzle = 128, int group = 1) {
            TmapSpec sp;
            sp.swizzle_bytes = swizzle;
            sp.base = base;
            sp.dtype = T.dtype;
            if (group > 1) {
                sp.rank = 5;
                sp.dims[0] = 64;
                sp.dims[1] = (uint64_t)sh[2];
                sp.dims[2] = (uint64_t)(sh[3] / 64);
                sp.dims[3] = (uint64_t)sh[1];
                sp.dims[4] = (uint64_t)sh[0];
                sp.strides_bytes[0] = (uint64_t)st[3] * es;
                sp.strides_bytes[1] = 128;
                sp.strides_bytes[2] = (uint64_t)st[2] * st[3] * es;
                sp.strides_bytes[3] = (uint64_t)st[1] * st[2] * st[3] * es;
                sp.box[0] = 64; sp.box[1] = box_rows; sp.box[2] = (uint32_t)group; sp.box[3] = 1; sp.box[4] = 1;
                env.encode_tmap(out, sp);
                return;
            }
            sp.dims[0] = (uint64_t)sh[3];
            sp.dims[1] = (uint64_t)sh[2];
            sp.dims[2] = (uint64_t)sh[1];
            sp.dims[3] = (uint64_t)sh[0];
            sp.strides_bytes[0] = (uint64_t)st[3] * es;
            sp.strides_bytes[1] = (uint64_t)st[2] * st[3] * es;
            sp.strides_bytes[2] = (uint64_t)st[1] * st[2] * st[3] * es;
            sp.box[0] = box_inner; sp.box[1] = box_rows; sp.box[2] = 1; sp.box[3] = 1;
            env.encode_tmap(out, sp);
        };
        // 1-D operands ([K] vectors) are viewed as one row / one column
        // K-major B role: one box holds the rows this CTA stages — all of the tile, or half in a pair
        const uint32_t b_rows = (uint32_t)(prog.pair_mode ? g.tile_n / 2 : g.tile_n);
        if (!swapped) {
            mk(A, ash, ast, pa, 64, g.a_mn_major ? 64 : 128, &g.tmA);
            mk(B, bsh, bst, pb, 64, g.b_mn_major ? 64 : b_rows, &g.tmB);
        } else {
            const int G = g.kgroup > 1 ? g.kgroup : 1;
            if (g.a_mn_major) mk(B, bsh, bst, pb, 64, 64 * G, &g.tmA);   // weights [K, N]: G k-blocks of a 64-wide chunk per box
            else mk(B, bsh, bst, pb, 64, 128, &g.tmA, 128, G);           // weights [N, K]
            mk(A, ash, ast, pa, 64, b_rows, &g.tmB, 128, G);             // activations
        }
        // ring: 16 KiB A block + this CTA's B block per stage, as many stages as fit in 192 KiB (at most 12)
        g.stage_b_bytes = (int32_t)(g.b_mn_major ? ((b_rows + 63) / 64) * 64 * 128 : b_rows * 128);
        if (swapped && g.kgroup > 1) g.stages = (int32_t)std::min<int64_t>(12, kSwappedRingBytes / (g.kgroup * (16 * 1024 + g.stage_b_bytes)));
        else g.stages = (int32_t)std::min<int64_t>(12, (192 * 1024) / ((g.tall ? 32 : 16) * 1024 + g.stage_b_bytes));
        // output through TMA stores of 32x32 blocks: needs 16-byte aligned rows and whole 32-column blocks per tile
        g.c_tma = (!swapped && g.c_vec && g.tile_n % 32 == 0 && (cst[3] * es) % 16 == 0 && (cst[2] * cst[3] * es) % 16 == 0 && !g.bias) ? 1 : 0;
        // The TMA-store epilogue (32x32 blocks through shared memory) keeps the accumulator hand-over short, which pays
        // when the main loop is long; its store rate is low (~0.45 TB/s over all SMs against ~1.4 TB/s for direct
        // stores), so tiles with a short K loop store directly. A fused all_reduce needs the TMA form.
        if (K < 8192 && !fuse_ar) g.c_tma = 0;
        if (g.c_tma) mk(C, csh, cst, pc, 32, 32, &g.tmC, 64);
        if (fuse_ar) {
            // Fused all_reduce: tiles go to the staging slots on the rank that sums their rows.
            const int R = env.nranks;
            if (!full || swapped || !g.c_tma || g.act != ACT_NONE || M % ((int64_t)R * tile_m) != 0)
                throw Error(E_UNSUPPORTED, "Matmul fused with AllReduce (one task) needs the full task range, TMA-aligned operands and "
                                           "M a multiple of 256 x world size");
            auto it = lay.coll_stage_offsets.find((int)fuse_ar->arg_int("Tag"));
            if (it == lay.coll_stage_offsets.end() || (int)it->second.size() != R)
                throw Error(E_PLAN, "fused AllReduce: staging slots were not published by every rank");
            g.peer_rows = (int32_t)(M / R);
            const uint64_t slot_bytes = (uint64_t)g.peer_rows * N * es;
            for (int r = 0; r < R; ++r) {
                TmapSpec sp;
                sp.swizzle_bytes = 64;
                sp.base = env.arena[r] + it->second[r] + (uint64_t)env.rank * slot_bytes;
                sp.dtype = C.dtype;
                sp.dims[0] = (uint64_t)N; sp.dims[1] = (uint64_t)g.peer_rows; sp.dims[2] = 1; sp.dims[3] = 1;
                sp.strides_bytes[0] = (uint64_t)N * es;
                sp.strides_bytes[1] = slot_bytes;
                sp.strides_bytes[2] = slot_bytes;
                sp.box[0] = 32; sp.box[1] = 32; sp.box[2] = 1; sp.box[3] = 1;
                env.encode_tmap(&g.tmPeer[r], sp);
            }
        }
        acc_begin();
        rd(A); rd_streamed(B);
        if (epi) rd(*epi);
        if (!swapped && full && g.splits <= 1 && !fuse_ar) {
            // tile -> CTA mapping of the output (and of an epilogue operand of the output's layout)
            uint64_t h = 1469598103934665603ull;
            for (int64_t v : {M, N, (int64_t)g.tile_n, (int64_t)g.tiles_m, (int64_t)g.tiles_n, (int64_t)g.raster_group, bn, bc, ldc,
                              (int64_t)g.c_stride_c, (int64_t)g.c_stride_n, (int64_t)g.tile_m})
                h = (h ^ (uint64_t)v) * 1099511628211ull;
            acc.tile_sig = h | 1;
            acc.tiled.push_back(span_of(C));
            if (epi && epi_mode != 2) acc.tiled.push_back(span_of(*epi));
        }
        if (g.splits > 1) wr_raw(g.ws, (size_t)g.splits * bn * bc * M * N * sizeof(float));
        else wr(C);
        if (fuse_ar) acc.opaque = true;  // tiles go to the peers' staging slots
        push(s, std::string("Matmul ") + op.name + " M=" + std::to_string(M) + " N=" + std::to_string(N) + " K=" +
                    std::to_string(K) + " tile_n=" + std::to_string(g.tile_n) + " units=" + std::to_string(g.n_units) +
                    (g.tall ? " tall" : "") + (g.plan_tiles ? " plan-tiles" : "") + (g.act ? " act=" + std::to_string(g.act) : "") +
                    (g.a_mn_major ? " A:MN" : " A:K") + (g.b_mn_major ? " B:MN" : " B:K") + (swapped ? " swapped" : "") +
                    (g.peer_rows ? " tiles->peer slots" : "") + (epi ? (epi_mode == 2 ? " rope" : epi_mode == 1 ? " *operand" : " +operand") : "") +
                    " stages=" + std::to_string(g.stages) + (g.kgroup > 1 ? "x" + std::to_string(g.kgroup) + "kb" : "") + (g.splits > 1 ? " splitK=" + std::to_string(g.splits) : ""));
        if (g.splits > 1) {
            // the activation and the rounding belong to the sum, not to the partials
            GemmArgs &gg = prog.stages.back().gm;
            const int act_final = gg.act;
            gg.act = ACT_NONE;
            gg.bias = nullptr;
            emit_sync(proc);
            Stage r = new_stage(SK_SPLITK_REDUCE, proc);
            SplitKReduceArgs &a = r.sr;
            a.C = pc;
            a.bias = (epi && epi_mode == 0) ? tensor_ptr(*epi) : nullptr;  // an added epilogue operand moves to the sum
            a.ws = gg.ws;
            a.ldc = ldc;
            a.c_stride_c = cst[2] * cst[3];
            a.c_stride_n = cst[1] * cst[2] * cst[3];
            a.M = (int32_t)M; a.N = (int32_t)N;
            a.batch_c = (int32_t)bc; a.batch_n = (int32_t)bn;
            a.splits = gg.splits;
            a.dtype = A.dtype;
            a.act = act_final;
            acc_begin();
            rd_raw(gg.ws, (size_t)gg.splits * bn * bc * M * N * sizeof(float));
            wr(C);
            push(r, "  split-K sum " + op.name + " splits=" + std::to_string(a.splits));
        }
    }

    // ---- decode attention -------------------------------------------------------------
    void lower_decode_attention(const OpDesc &op, const Range &proc) {
        const TensorDesc &q = op.reads.at(0), &k = op.reads.at(1), &v = op.reads.at(2), &o = op.results.at(0);
        auto qs = q.shape4(), ks = k.shape4(), vs = v.shape4(), os = o.shape4();
        auto qst = q.strides4(), kst = k.strides4(), vst = v.strides4(), ost = o.strides4();
        const int64_t B = qs[0], Hq = qs[1], Hkv = ks[1], T = ks[2], D = qs[3];
        if (q.dtype != k.dtype || q.dtype != v.dtype || q.dtype != o.dtype || (q.dtype != DT_F16 && q.dtype != DT_BF16))
            throw Error(E_UNSUPPORTED, "DecodeAttention: fp16 or bf16 operands of one type");
        if (D != 128 || qs[2] != 1 || ks[3] != D || vs[3] != D || ks[0] != B || vs[0] != B || vs[1] != Hkv || vs[2] != T || os != qs)
            throw Error(E_UNSUPPORTED, "DecodeAttention: q [B, Hq, 1, 128], k and v [B, Hkv, T, 128]");
        const int64_t G = Hkv > 0 ? Hq / Hkv : 0;
        if (Hkv <= 0 || Hq % Hkv || !(G == 1 || G == 2 || G == 4 || G == 8))
            throw Error(E_UNSUPPORTED, "DecodeAttention: 1, 2, 4 or 8 query heads per K/V head");
        Stage s = new_stage(SK_DECODE_ATTN, proc);
        DecodeAttnArgs &a = s.da;
        a.out = tensor_ptr(o); a.q = tensor_ptr(q); a.k = tensor_ptr(k); a.v = tensor_ptr(v);
        a.q_stride_h = qst[2] * qst[3]; a.q_stride_b = qst[1] * qst[2] * qst[3];
        const OpDesc *rope = rope_for_attention;
        rope_for_attention = nullptr;
        if (rope) {
            // the unrotated query (dense, the rotated one's layout) and the position's table take the place of q
            if (rope->results[0].buffer_id != q.buffer_id || !q.dense() || !rope->reads[0].dense())
                throw Error(E_INTERNAL, "rotary embedding folded into an attention that does not read it");
            a.q = tensor_ptr(rope->reads[0]);
            a.rope = tensor_ptr(rope->reads[1]);
            if (!aligned16(a.rope)) throw Error(E_UNSUPPORTED, "DecodeAttention: the rotary table must be 16-byte aligned");
        }
        a.o_stride_h = ost[2] * ost[3]; a.o_stride_b = ost[1] * ost[2] * ost[3];
        a.k_ld = kst[3]; a.k_stride_h = kst[2] * kst[3]; a.k_stride_b = kst[1] * kst[2] * kst[3];
        a.v_ld = vst[3]; a.v_stride_h = vst[2] * vst[3]; a.v_stride_b = vst[1] * vst[2] * vst[3];
        if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || a.k_ld % 8 || a.v_ld % 8 || a.q_stride_h % 8 || a.q_stride_b % 8 ||
            a.k_stride_h % 8 || a.k_stride_b % 8 || a.v_stride_h % 8 || a.v_stride_b % 8)
            throw Error(E_UNSUPPORTED, "DecodeAttention: rows must be 16-byte aligned");
        a.B = (int32_t)B; a.Hq = (int32_t)Hq; a.Hkv = (int32_t)Hkv; a.T = (int32_t)T;
        a.dtype = q.dtype;
        a.scale = op.has_arg("Scale") ? (float)op.arg_float("Scale") : 1.0f;
        // chunks of the cache: at most two work items per CTA (one more would cost a third round), at least 128 and at
        // most 2048 keys each; among the candidates the one with the least makespan (rounds x keys per item)
        const int64_t P = proc.count();
        const int64_t max_chunks = std::max<int64_t>(1, std::min<int64_t>(2 * P / (B * Hkv), (T + 127) / 128));
        int64_t chunks = 1, chunk_len = 0;
        {
            int64_t best = -1;
            for (int64_t c = 1; c <= max_chunks; ++c) {
                const int64_t len = std::min<int64_t>(2048, ((T + c - 1) / c + 31) / 32 * 32);
                const int64_t n = (T + len - 1) / len;
                const int64_t rounds = (B * Hkv * n + P - 1) / P;
                const int64_t cost = rounds * (len + 64);  // 64 keys' worth of fixed cost per item
                if (best < 0 || cost < best) { best = cost; chunks = n; chunk_len = len; }
            }
        }
        a.chunks = (int32_t)chunks; a.chunk_len = (int32_t)chunk_len;
        const size_t bytes = (size_t)B * Hkv * chunks * G * (128 + 2) * sizeof(float);
        a.ws = env.workspace ? reinterpret_cast<float *>(env.workspace + prog.workspace_bytes) : nullptr;
        prog.workspace_bytes += (bytes + 255) / 256 * 256;
        a.phase = 0;
        acc_begin();
        if (rope) { rd(rope->reads[0]); rd(rope->reads[1]); } else rd(q);
        rd_streamed(k); rd_streamed(v);
        wr_raw(a.ws, bytes);
        push(s, "DecodeAttention " + op.name + " B=" + std::to_string(B) + " heads=" + std::to_string(Hq) + "/" + std::to_string(Hkv) +
                    " keys=" + std::to_string(T) + " chunks=" + std::to_string(chunks) + " x " + std::to_string(chunk_len) + (rope ? " <-rope" : ""));
        // When the only reader of the result is the weight-streaming matmul of the next processor group (one or two
        // sequences), that stage merges the chunks while it stages its activations: no merge stage, one barrier less.
        if (fold_decode_chain() && env.workspace) {
            const TaskGroup *ntg = nullptr;
            const OpDesc *nx = first_op_of(cur_pg + 1, &ntg);
            if (nx && nx->type == "Matmul" && !nx->reads.empty() && nx->reads[0].buffer_id == o.buffer_id && nx->reads[0].dense() &&
                nx->reads[0].shape4()[2] == B && nx->reads[0].shape4()[3] == Hq * 128 && o.dense() && matmul_is_gemv(*nx, *ntg) &&
                other_readers(o.buffer_id, nx) == 0) {
                pending_merge.buffer_id = o.buffer_id;
                pending_merge.ws = a.ws; pending_merge.ws_bytes = bytes;
                pending_merge.chunks = (int)chunks; pending_merge.group = (int)G; pending_merge.kv_heads = (int)Hkv;
                pending_merge.B = B; pending_merge.Hq = Hq;
                pending_merge_pg = cur_pg;
                return;
            }
        }
        emit_sync(proc);
        Stage m = s;
        m.da.phase = 1;
        acc_begin();
        rd_raw(a.ws, bytes);
        wr(o);
        push(m, "  merge of the chunks " + op.name);
    }

    // ---- prefill attention ----------------------------------------------------------------
    // q [B, Hq, Tq, 128], k and v [B, Hkv, Tkv, 128], out as q; with "TokenMajor": 1 all four have the head and token
    // axes exchanged ([B, T, H, 128], the layout the projections produce).
    void lower_prefill_attention(const OpDesc &op, const Range &proc) {
        const TensorDesc &q = op.reads.at(0), &k = op.reads.at(1), &v = op.reads.at(2), &o = op.results.at(0);
        if (q.dtype != k.dtype || q.dtype != v.dtype || q.dtype != o.dtype || (q.dtype != DT_F16 && q.dtype != DT_BF16))
            throw Error(E_UNSUPPORTED, "PrefillAttention: fp16 or bf16 operands of one type");
        if (prog.pair_mode) throw Error(E_UNSUPPORTED, "PrefillAttention: not available in a plan lowered for CTA pairs");
        if (!env.encode_tmap) throw Error(E_UNSUPPORTED, "PrefillAttention: needs tensor maps");
        const bool bthd = op.has_arg("TokenMajor") && op.arg_int("TokenMajor") != 0;
        const std::string layout = bthd ? "bthd" : "bhtd";
        const int hx = bthd ? 2 : 1, tx = bthd ? 1 : 2;  // which axis holds heads / tokens
        auto qs = q.shape4(), ks = k.shape4(), vs = v.shape4(), os = o.shape4();
        const int64_t B = qs[0], Hq = qs[hx], Tq = qs[tx], Hkv = ks[hx], Tkv = ks[tx];
        if (qs[3] != 128 || ks[3] != 128 || vs != ks || os != qs || ks[0] != B || Hkv <= 0 || Hq % Hkv || Tq <= 0 || Tkv <= 0)
            throw Error(E_UNSUPPORTED, "PrefillAttention: q [B, Hq, Tq, 128], k and v [B, Hkv, Tkv, 128], Hq a multiple of Hkv");
        const int es = 2;
        // element strides of the (b, h, t) axes of a tensor
        auto strides = [&](const TensorDesc &T, int64_t &sb, int64_t &sh, int64_t &st) {
            auto s4 = T.strides4();
            const int64_t s1 = s4[2] * s4[3], s2 = s4[3];
            sb = s4[1] * s4[2] * s4[3];
            sh = bthd ? s2 : s1;
            st = bthd ? s1 : s2;
        };
        Stage s = new_stage(SK_PREFILL_ATTN, proc);
        PrefillAttnArgs &a = s.pa;
        auto mk = [&](const TensorDesc &T, int64_t H, int64_t Tn, uint32_t box_rows, CUtensorMap *out, const char *what) {
            int64_t sb, sh, st;
            strides(T, sb, sh, st);
            char *base = tensor_ptr(T);
            if (!aligned16(base) || (st * es) % 16 || (sh * es) % 16 || (sb * es) % 16)
                throw Error(E_UNSUPPORTED, std::string("PrefillAttention: ") + what + " rows must be 16-byte aligned");
            TmapSpec sp;
            sp.base = base;
            sp.dtype = T.dtype;
            sp.dims[0] = 128; sp.dims[1] = (uint64_t)Tn; sp.dims[2] = (uint64_t)H; sp.dims[3] = (uint64_t)B;
            sp.strides_bytes[0] = (uint64_t)st * es; sp.strides_bytes[1] = (uint64_t)sh * es; sp.strides_bytes[2] = (uint64_t)sb * es;
            sp.box[0] = 64; sp.box[1] = box_rows; sp.box[2] = 1; sp.box[3] = 1;
            env.encode_tmap(out, sp);
        };
        mk(q, Hq, Tq, 128, &a.tmQ, "q");
        mk(k, Hkv, Tkv, 128, &a.tmK, "k");
        mk(v, Hkv, Tkv, 64, &a.tmV, "v");
        a.out = tensor_ptr(o);
        strides(o, a.o_stride_b, a.o_stride_h, a.o_stride_t);
        if (!aligned16(a.out) || a.o_stride_t % 8 || a.o_stride_h % 8 || a.o_stride_b % 8)
            throw Error(E_UNSUPPORTED, "PrefillAttention: output rows must be 16-byte aligned");
        a.B = (int32_t)B; a.Hq = (int32_t)Hq; a.Hkv = (int32_t)Hkv; a.Tq = (int32_t)Tq; a.Tkv = (int32_t)Tkv;
        a.causal = op.has_arg("Causal") ? (int32_t)op.arg_int("Causal") : 0;
        a.dtype = q.dtype;
        a.scale = op.has_arg("Scale") ? (float)op.arg_float("Scale") : 1.0f;
        if (!(a.scale > 0.0f)) throw Error(E_UNSUPPORTED, "PrefillAttention: Scale must be positive");
        a.q_tiles = (int32_t)((Tq + 127) / 128);
        a.n_units = (int32_t)(B * Hq * a.q_tiles);
        const TensorDesc *mask = op.reads.size() > 3 ? &op.reads[3] : nullptr;
        if (mask) {
            auto ms = mask->shape4();
            auto mst = mask->strides4();
            if (mask->dtype != q.dtype || ms[2] != Tq || ms[3] != Tkv || (ms[0] != 1 && ms[0] != B) || (ms[1] != 1 && ms[1] != Hq))
                throw Error(E_UNSUPPORTED, "PrefillAttention: mask [B or 1, Hq or 1, Tq, Tkv] of the operands' type");
            a.mask = tensor_ptr(*mask);
            a.m_stride_q = mst[3];
            a.m_stride_h = ms[1] == 1 ? 0 : mst[2] * mst[3];
            a.m_stride_b = ms[0] == 1 ? 0 : mst[1] * mst[2] * mst[3];
            if (!aligned16(a.mask) || a.m_stride_q % 8 || a.m_stride_h % 8 || a.m_stride_b % 8)
                throw Error(E_UNSUPPORTED, "PrefillAttention: mask rows must be 16-byte aligned");
        }
        acc_begin();
        rd(q); rd(k); rd(v);
        if (mask) rd(*mask);
        wr(o);
        push(s, "PrefillAttention " + op.name + " B=" + std::to_string(B) + " heads=" + std::to_string(Hq) + "/" + std::to_string(Hkv) +
                    " rows=" + std::to_string(Tq) + " keys=" + std::to_string(Tkv) + (a.causal ? " causal" : "") + (mask ? " +mask" : "") + " " + layout +
                    " units=" + std::to_string(a.n_units));
    }

    // ---- transpose / embedding ---------------------------------------------------------
    void lower_transpose(const OpDesc &op, const Range &proc, const TaskGroup &tg) {
        const bool partial = !full_range(tg.task_range, num_tasks(op));
        const TensorDesc &in = op.reads.at(0), &out = op.results.at(0);
        auto perm = op.arg_dims("Permutation");
        const int nd = (int)in.shape.size();
        if ((int)perm.size() != nd) throw Error(E_MODEL, "Transpose: permutation rank mismatch");
        Stage s = new_stage(SK_TRANSPOSE, proc);
        TransposeArgs &a = s.tp;
        acc_begin();
        rd(in);
        wr(out);
        a.in = make_ref(in);
        a.out = make_ref(out);
        for (int i = 0; i < 4 - nd; ++i) a.perm[i] = i;
        for (int i = 0; i < nd; ++i) a.perm[4 - nd + i] = (int32_t)perm[i] + 4 - nd;
        for (int i = 0; i < 4; ++i)
            if (a.out.shape[i] != a.in.shape[a.perm[i]]) throw Error(E_MODEL, "Transpose: output shape mismatch");
        const int V = (int)(16 / dtype_size(in.dtype));
        bool vec = a.perm[3] == 3 && aligned16(a.in.ptr) && aligned16(a.out.ptr) && a.out.shape[3] % V == 0;
        for (int i = 0; i < 3; ++i) vec = vec && a.in.stride[i] % V == 0 && a.out.stride[i] % V == 0;
        a.out.contiguous = vec ? 2 : a.out.contiguous;
        if (partial) {
            if (!op.config.is_object() || !op.config.contains("Tile")) throw Error(E_PLAN, "Transpose: a partial TaskRange needs the Tile of the tasks");
            auto tile = op.config.at("Tile").as_int_vec();
            if (tile.size() != 2 || tile[0] <= 0 || tile[1] <= 0) throw Error(E_PLAN, "Transpose: Tile should have 2 positive elements");
            a.partial = 1;
            a.tile_h = (int32_t)tile[0]; a.tile_w = (int32_t)tile[1];
            a.task_b = tg.task_range.b; a.task_e = tg.task_range.e; a.task_s = std::max<int64_t>(1, tg.task_range.s);
        }
        push(s, "Transpose " + op.name + (vec && !partial ? " vec" : "") +
                    (partial ? " tasks [" + std::to_string(a.task_b) + "," + std::to_string(a.task_e) + (a.task_s != 1 ? "," + std::to_string(a.task_s) : "") + ")" : ""));
    }

    void lower_embedding(const OpDesc &op, const Range &proc, const TaskGroup &tg) {
        const bool partial = !full_range(tg.task_range, num_tasks(op));
        const TensorDesc &idx = op.reads.at(0), &w = op.reads.at(1), &out = op.results.at(0);
        if (idx.dtype != DT_I32) throw Error(E_MODEL, "Embedding: indices must be INT32");
        if (!idx.dense()) throw Error(E_UNSUPPORTED, "Embedding: strided index tensor");
        auto osh = out.shape4(), ost = out.strides4(), wsh = w.shape4(), wst = w.strides4();
        if (!((osh[0] * osh[1] == 1 || ost[2] == osh[2]) && (osh[0] == 1 || ost[1] == osh[1])))
            throw Error(E_UNSUPPORTED, "Embedding: output rows must be evenly spaced");
        Stage s = new_stage(SK_EMBED, proc);
        EmbedArgs &a = s.em;
        acc_begin();
        rd(idx); rd(w);
        wr(out);
        a.out = tensor_ptr(out);
        a.idx = reinterpret_cast<const int32_t *>(tensor_ptr(idx));
        a.weight = tensor_ptr(w);
        a.n_idx = idx.nelems();
        a.num_emb = wsh[2];
        a.emb_dim = wsh[3];
        a.w_ld = wst[3];
        a.out_ld = ost[3];
        a.esize = (int32_t)dtype_size(w.dtype);
        a.task_b = 0; a.task_s = 1;
        if (partial) {
            // a task gathers one row (ark/ops/ops_embedding.cpp: NumTasks = indices)
            if (num_tasks(op) != idx.nelems()) throw Error(E_UNSUPPORTED, "Embedding: a partial TaskRange needs one task per index");
            const int64_t e = std::min<int64_t>(tg.task_range.e, idx.nelems());
            a.task_b = tg.task_range.b; a.task_s = std::max<int64_t>(1, tg.task_range.s);
            a.n_idx = e > a.task_b ? (e - a.task_b + a.task_s - 1) / a.task_s : 0;
        }
        push(s, "Embedding " + op.name + " n=" + std::to_string(a.n_idx) +
                    (partial ? " tasks from " + std::to_string(a.task_b) + " step " + std::to_string(a.task_s) : ""));
    }

    // ---- communication ------------------------------------------------------------------
    static int channel_of(int tag) { return (int)(((uint32_t)tag) % kChannels); }

    void lower_send(const OpDesc &op, const Range &proc) {
        const TensorDesc &src = op.reads.at(0), &dst = op.writes.at(0);
        const int peer = dst.buffer_rank;
        if (peer < 0 || peer >= env.nranks || peer == env.rank) throw Error(E_MODEL, "Send: invalid remote rank");
        if (!src.dense() || !dst.dense() || src.nelems() != dst.nelems() || src.dtype != dst.dtype)
            throw Error(E_UNSUPPORTED, "Send: dense tensors of equal size only");
        if (dst.recv_tags.empty()) throw Error(E_MODEL, "Send: destination buffer carries no tag");
        Stage s = new_stage(SK_PUT, proc);
        s.put.dst = tensor_ptr(dst);
        s.put.src = tensor_ptr(src);
        s.put.bytes = src.nelems() * (int64_t)dtype_size(src.dtype);
        s.put.peer = peer;
        s.put.iter_slots = (int32_t)config_int(op, "IterSlots", 1);
        s.put.src_iter_bytes = config_int(op, "InIterStride", 0) * (int64_t)dtype_size(src.dtype);
        push(s, "Send " + op.name + " -> rank " + std::to_string(peer) + " bytes=" + std::to_string(s.put.bytes));
        const bool signal = !op.config.is_object() || !op.config.contains("Signal") || op.config.at("Signal").as_bool();
        if (signal) {
            emit_sync(proc);
            Stage g = new_stage(SK_SIGNAL, proc);
            g.sg.peer = peer;
            g.sg.channel = channel_of(dst.recv_tags[0].second);
            push(g, "  signal rank " + std::to_string(peer) + " ch " + std::to_string(g.sg.channel));
        }
    }

    void lower_recv(const OpDesc &op, const Range &proc) {
        const TensorDesc &stand_in = op.reads.at(0);
        const int peer = stand_in.buffer_rank;
        if (peer < 0 || peer >= env.nranks || peer == env.rank) throw Error(E_MODEL, "Recv: invalid remote rank");
        const bool wait = !op.config.is_object() || !op.config.contains("Wait") || op.config.at("Wait").as_bool();
        if (!wait) return;  // placeholder op expressing a dependency only (ops_all_reduce_test.cpp:210-215)
        if (stand_in.send_tags.empty()) throw Error(E_MODEL, "Recv: source buffer carries no tag");
        Stage s = new_stage(SK_WAITFLAG, proc);
        s.wt.peer = peer;
        s.wt.channel = channel_of(stand_in.send_tags[0].second);
        push(s, "Recv " + op.name + " <- rank " + std::to_string(peer) + " ch " + std::to_string(s.wt.channel));
    }

    // ---- packets (SendPacket / RecvPacket / RecvReduceSendPacket) and RecvReduceSend ----------------------
    // ark/ops/ops_communication.cpp:171-560. Packet tensors are UINT8 views twice the size of their payload.
    static int64_t dense_bytes(const TensorDesc &t, const char *what) {
        if (!t.dense()) throw Error(E_UNSUPPORTED, std::string(what) + ": dense tensors only");
        return t.nelems() * (int64_t)dtype_size(t.dtype);
    }
    void check_full(const OpDesc &op, const TaskGroup &tg) const {
        if (!full_range(tg.task_range, num_tasks(op))) throw Error(E_UNSUPPORTED, op.type + ": partial TaskRange is not supported");
    }
    uint32_t flag_of(const OpDesc &op) const { return op.has_arg("Flag") ? (uint32_t)op.arg_int("Flag") : 1u; }

    void lower_send_packet(const OpDesc &op, const Range &proc, const TaskGroup &tg) {
        check_full(op, tg);
        const TensorDesc &src = op.reads.at(0), &dst = op.writes.at(0);
        const int peer = dst.buffer_rank;
        if (peer < 0 || peer >= env.nranks || peer == env.rank) throw Error(E_MODEL, "SendPacket: invalid remote rank");
        const int64_t payload = dense_bytes(src, "SendPacket");
        if (dense_bytes(dst, "SendPacket") != 2 * payload) throw Error(E_MODEL, "SendPacket: the packet tensor must be twice the payload");
        Stage s = new_stage(SK_PACKET, proc);
        s.pk.dst = tensor_ptr(dst);
        s.pk.src = tensor_ptr(src);
        s.pk.payload_bytes = payload;
        s.pk.flag = flag_of(op);
        s.pk.get = 0;
        if (payload % 8 || !aligned16(s.pk.dst) || (reinterpret_cast<uintptr_t>(s.pk.src) & 7))
            throw Error(E_UNSUPPORTED, "SendPacket: payload must be a multiple of 8 bytes, 8-byte aligned, the packet buffer 16-byte aligned");
        push(s, "SendPacket " + op.name + " -> rank " + std::to_string(peer) + " payload=" + std::to_string(payload));
    }

    void lower_recv_packet(const OpDesc &op, const Range &proc, const TaskGroup &tg) {
        check_full(op, tg);
        const TensorDesc &scratch = op.reads.at(1), &out = op.writes.at(0);  // reads[0] only names the sender
        const int64_t payload = dense_bytes(out, "RecvPacket");
        if (dense_bytes(scratch, "RecvPacket") != 2 * payload) throw Error(E_MODEL, "RecvPacket: the packet tensor must be twice the payload");
        Stage s = new_stage(SK_PACKET, proc);
        s.pk.dst = tensor_ptr(out);
        s.pk.src = tensor_ptr(scratch);
        s.pk.payload_bytes = payload;
        s.pk.flag = flag_of(op);
        s.pk.get = 1;
        if (payload % 8 || !aligned16(s.pk.src) || (reinterpret_cast<uintptr_t>(s.pk.dst) & 7))
            throw Error(E_UNSUPPORTED, "RecvPacket: payload must be a multiple of 8 bytes, 8-byte aligned, the packet buffer 16-byte aligned");
        push(s, "RecvPacket " + op.name + " <- rank " + std::to_string(op.reads.at(0).buffer_rank) + " payload=" + std::to_string(payload));
    }

    void lower_recv_reduce_send(const OpDesc &op, const Range &proc, const TaskGroup &tg, bool packets) {
        check_full(op, tg);
        const TensorDesc &in = op.reads.at(0), &scratch = op.reads.at(1), &out = op.writes.at(0);
        const int npeers = (int)op.arg_int("NPeers");
        if (npeers < 1 || npeers >= kMaxPeers || (int)op.writes.size() != npeers + 1)
            throw Error(E_MODEL, op.type + ": one output tensor per peer expected");
        if (!(in.dtype == DT_F32 || in.dtype == DT_F16 || in.dtype == DT_BF16) || out.dtype != in.dtype)
            throw Error(E_UNSUPPORTED, op.type + ": floating-point tensors of one type");
        const int64_t bytes = dense_bytes(in, op.type.c_str());
        if (dense_bytes(out, op.type.c_str()) != bytes) throw Error(E_MODEL, op.type + ": input and output sizes differ");
        if (dense_bytes(scratch, op.type.c_str()) != bytes * npeers * (packets ? 2 : 1))
            throw Error(E_MODEL, op.type + ": scratch must hold one shard per peer");
        Stage s = new_stage(SK_PACKET_REDUCE, proc);
        PacketReduceArgs &a = s.pr;
        a.in = tensor_ptr(in);
        a.out = tensor_ptr(out);
        a.scratch = tensor_ptr(scratch);
        a.nelem = in.nelems();
        a.dtype = in.dtype;
        a.npeers = npeers;
        a.packets = packets ? 1 : 0;
        a.flag = flag_of(op);
        bool ok = aligned16(a.scratch) && bytes % (packets ? 8 : 16) == 0 &&
                  (reinterpret_cast<uintptr_t>(a.in) & (packets ? 7 : 15)) == 0 && (reinterpret_cast<uintptr_t>(a.out) & (packets ? 7 : 15)) == 0;
        for (int q = 0; q < npeers; ++q) {
            const TensorDesc &po = op.writes[q + 1];
            if (dense_bytes(po, op.type.c_str()) != bytes * (packets ? 2 : 1)) throw Error(E_MODEL, op.type + ": peer output size mismatch");
            a.peer_out[q] = tensor_ptr(po);
            ok = ok && aligned16(a.peer_out[q]);
        }
        if (!ok) throw Error(E_UNSUPPORTED, op.type + ": shards must be 16-byte aligned and a multiple of 16 bytes (8 with packets)");
        push(s, op.type + " " + op.name + " peers=" + std::to_string(npeers) + " bytes=" + std::to_string(bytes) + (packets ? " packets" : ""));
    }

    bool same_offset_everywhere(const AllReduceArgs &a) const {
        for (int r = 1; r < env.nranks; ++r)
            if (a.buf_off[r] != a.buf_off[0]) return false;
        return true;
    }

    void emit_peersync(const Range &proc, const std::string &why) {
        Stage s = new_stage(SK_PEERSYNC, proc);
        s.ps.ord = ++prog.peersyncs_per_iter;
        push(s, "peer barrier #" + std::to_string(s.ps.ord) + " (" + why + ")");
    }

    // Grid barrier, exchange with the peers, grid barrier: one stage when the range is a dense run of CTAs starting at
    // CTA 0 of the range (CTA 0 does the exchange between the two halves of the barrier), three stages otherwise.
    void emit_grid_peer_barrier(const Range &proc, const std::string &why) {
        static const bool merged = []() { const char *e = getenv("ARKB_MERGED_PEER_BARRIER"); return e ? atoi(e) != 0 : true; }();
        if (!merged || proc.s != 1 || proc.count() < 2) {
            emit_sync(proc);
            emit_peersync(proc, why);
            emit_sync(proc);
            return;
        }
        auto key = std::make_tuple(proc.b, proc.e, (int64_t)-1);  // a counter of its own: it advances by CTAs + 1
        auto it = sync_ids.find(key);
        int id;
        if (it == sync_ids.end()) {
            id = (int)sync_ids.size();
            if (id >= kMaxSyncGroups - 1) throw Error(E_UNSUPPORTED, "too many distinct processor ranges need a barrier");
            sync_ids[key] = id;
        } else {
            id = it->second;
        }
        Stage s = new_stage(SK_PEERSYNC, proc);
        s.ps.ord = ++prog.peersyncs_per_iter;
        s.ps.with_grid = 1;
        s.sync_group = id;
        s.sync_count = (int32_t)proc.count() + 1;
        s.sync_ord = ++prog.syncs_per_iter[id];
        acc_begin();  // touches no tensor; the dependency pass treats it as a whole-range barrier
        push(s, "grid + peer barrier #" + std::to_string(s.ps.ord) + " (" + why + ")");
    }

    void lower_device_sync(const OpDesc &op, const Range &proc) {
        if (env.nranks == 1) return;
        emit_grid_peer_barrier(proc, "DeviceSync " + op.name);
    }

    // fused: the partials already sit in this rank's staging slots (put there by every rank's Matmul epilogue)
    // pushed: the matmul before it (same task) has already stored its result into every rank's staging slot
    // add: the Add of the same task that consumes the sum (one-shot only): folded into the reduce phase
    void lower_all_reduce(const OpDesc &op, const Range &proc, bool fused = false, bool pushed = false, const OpDesc *add = nullptr) {
        if (env.nranks == 1) return;
        const TensorDesc &t = op.results.at(0);
        if (!t.dense()) throw Error(E_UNSUPPORTED, "AllReduce: dense tensors only");
        const int tag = (int)op.arg_int("Tag");
        auto it = lay.coll_offsets.find(tag);
        if (it == lay.coll_offsets.end() || (int)it->second.size() != env.nranks)
            throw Error(E_PLAN, "AllReduce: tag " + std::to_string(tag) + " was not published by every rank");
        const size_t es = dtype_size(t.dtype);
        const int V = (int)(16 / es);
        const int64_t n = t.nelems();
        const size_t bytes = (size_t)n * es;
        Stage s = new_stage(SK_ALLREDUCE, proc);
        AllReduceArgs &a = s.ar;
        for (int r = 0; r < env.nranks; ++r) {
            a.buf_off[r] = it->second[r];
            if (a.buf_off[r] % 16) throw Error(E_UNSUPPORTED, "AllReduce: tensor must be 16-byte aligned");
        }
        if (n % V) throw Error(E_UNSUPPORTED, "AllReduce: element count must be a multiple of 16 bytes");
        a.nelem = n;
        a.dtype = t.dtype;
        std::string algo = op.config.is_object() && op.config.contains("Algo") ? op.config.at("Algo").as_string() : "auto";
        // Gather = false: every rank keeps only the sum of its own 1/p of the rows (what a host that reads the result
        // shard by shard needs); only the form fused with the producing Matmul offers it
        const bool gather = !(op.has_arg("Gather") && !op.arg_bool("Gather"));
        if (!gather && !fused) throw Error(E_UNSUPPORTED, "AllReduce without gather needs the form fused with the Matmul before it");
        if (fused) {
            auto st = lay.coll_stage_offsets.find(tag);
            if (st == lay.coll_stage_offsets.end()) throw Error(E_PLAN, "fused AllReduce: no staging slots");
            if (n % ((int64_t)V * env.nranks)) throw Error(E_UNSUPPORTED, "fused AllReduce: size must split evenly over the ranks");
            a.algo = 2;
            a.stage_off = st->second[env.rank];
            a.stage_bytes = bytes / env.nranks;
            a.no_gather = gather ? 0 : 1;
            a.mc_store = (gather && env.mc_arena && same_offset_everywhere(a)) ? 1 : 0;
            emit_grid_peer_barrier(proc, "partial tiles pushed");
            push(s, "AllReduce " + op.name + (gather ? (a.mc_store ? " sum of staging slots + multicast store bytes=" : " sum of staging slots + all-gather bytes=")
                                                 : " sum of staging slots, own rows only bytes=") + std::to_string(bytes));
            emit_grid_peer_barrier(proc, "all_reduce outputs stored");
            return;
        }
        const size_t slot = lay.comm_stage_bytes / kMaxPeers;
        const bool one = (algo == "oneshot") || (algo == "auto" && bytes <= 256 * 1024);
        if (one && bytes > slot) throw Error(E_PLAN, "AllReduce: tensor exceeds the one-shot staging area");
        if (one) {
            a.algo = 0;
            a.stage_bytes = lay.comm_stage_bytes;
            a.ord = oneshot_ord++;
            a.phase = 0;
            if (!pushed) push(s, "AllReduce " + op.name + " one-shot push bytes=" + std::to_string(bytes));
            emit_grid_peer_barrier(proc, "all_reduce data pushed");
            {
                // the consumers add the slots up themselves when they are the weight-streaming matmuls that open the next
                // processor group(s) and the tensor is one or two dense rows
                const TensorDesc &res = add ? add->results.at(0) : t;
                auto rs = res.shape4();
                if (fold_decode_chain() && res.dense() && t.dense() && rs[0] * rs[1] == 1 && rs[2] <= kGemvMaxM && rs[3] % 8 == 0 &&
                    res.nelems() == t.nelems() && sum_consumer(cur_pg + 1, res.buffer_id, rs[2], rs[3])) {
                    pending_sum = PendingSum();
                    pending_sum.buffer_id = res.buffer_id;
                    pending_sum.ord = a.ord + 1;
                    pending_sum.out = res;
                    pending_sum.rows = rs[2]; pending_sum.cols = rs[3];
                    if (add) {
                        pending_sum.has_residual = true;
                        pending_sum.residual = add->reads[0].id == t.id ? add->reads[1] : add->reads[0];
                    }
                    if (!add || (pending_sum.residual.dense() && pending_sum.residual.nelems() == res.nelems() &&
                                 pending_sum.residual.dtype == res.dtype)) {
                        prog.notes.back() += " (sum left to the consumers)";
                        return;
                    }
                    pending_sum = PendingSum();
                }
            }
            Stage s2 = s;
            s2.ar.phase = 1;
            if (add) {
                const TensorDesc &other = add->reads[0].id == t.id ? add->reads[1] : add->reads[0];
                s2.ar.residual = tensor_ptr(other);
                s2.ar.sum_out = tensor_ptr(add->results.at(0));
                if (!aligned16(s2.ar.residual) || !aligned16(s2.ar.sum_out)) throw Error(E_UNSUPPORTED, "AllReduce + Add: operands must be 16-byte aligned");
            }
            push(s2, "AllReduce " + op.name + " one-shot reduce" + (add ? " +residual" : ""));
        } else {
            // NVLS when the arenas are bound to a multicast object (the executor was asked for it) and the tensor has
            // one offset on all ranks; "Algo": "twoshot" keeps the peer loads and stores
            // (with 2 ranks the switch path moves more bytes per GPU than the direct exchange: 1.5 S against 1.0 S out,
            // measured 395 against 631 GB/s at 256 MiB; from 4 ranks on it moves fewer, 1.125 S against 1.75 S at 8)
            const bool nvls = env.mc_arena && same_offset_everywhere(a) && (algo == "nvls" || (algo == "auto" && env.nranks >= 4));
            if (algo == "nvls" && !nvls) throw Error(E_UNSUPPORTED, "AllReduce: NVLS needs a multicast-bound arena (ARKB_NVLS=1) and one tensor offset on all ranks");
            a.algo = nvls ? 3 : 1;
            emit_grid_peer_barrier(proc, "all_reduce inputs ready");
            push(s, "AllReduce " + op.name + (nvls ? " NVLS (multimem.ld_reduce + multimem.st) bytes=" : " two-shot bytes=") + std::to_string(bytes));
            emit_grid_peer_barrier(proc, "all_reduce outputs stored");
        }
    }

    // ---- op chains the reference composes for softmax / layernorm / rmsnorm -> one row kernel --------------
    // Unmodified reference models emit these as 5-7 operators (python/ark/ops.py:491-513,
    // examples/llama/model.py:92-99); run one after the other each costs a pass over the tensor and a barrier. When
    // the operators follow each other (inside one task, or as consecutive single-operator processor groups) and
    // nothing else reads the intermediates, the chain is lowered to the fused row kernel instead.
    bool private_to(const TensorDesc &t, const std::vector<const OpDesc *> &chain, int64_t out_buffer) const {
        if (t.buffer_id == out_buffer) return true;  // in-place chains: outsiders see the final value
        for (auto &ti : plan.task_infos)
            for (auto &o : ti.ops) {
                if (std::find(chain.begin(), chain.end(), &o) != chain.end()) continue;
                for (auto &rd : o.reads)
                    if (rd.buffer_id == t.buffer_id) return false;
            }
        return true;
    }
    static bool last_axis(const OpDesc &op) {
        if (!op.has_arg("Axis") || op.reads.empty()) return false;
        const int nd = (int)op.reads[0].shape.size();
        int ax = (int)op.arg_int("Axis");
        if (ax < 0) ax += nd;
        return ax == nd - 1;
    }
    static bool reads_ids(const OpDesc &op, int64_t a, int64_t b = -1) {
        if (b < 0) return op.reads.size() == 1 && op.reads[0].id == a;
        return op.reads.size() == 2 && op.reads[0].id == a && op.reads[1].id == b;
    }
    static bool fp_type(int dt) { return dt == DT_F32 || dt == DT_F16 || dt == DT_BF16; }

    // Tries to match a chain starting at seq[i]; on success fills `fused` (a RowOp operator) and returns its length.
    size_t match_chain(const std::vector<const OpDesc *> &seq, size_t i, OpDesc &fused) const {
        if (const char *e = getenv("ARKB_FUSE_CHAINS")) if (!atoi(e)) return 0;
        auto T = [&](size_t k) -> const OpDesc & { return *seq[i + k]; };
        auto have = [&](size_t n) { return i + n <= seq.size(); };
        auto res = [&](size_t k) -> const TensorDesc & { return T(k).results.at(0); };
        auto chain_of = [&](size_t n) { return std::vector<const OpDesc *>(seq.begin() + i, seq.begin() + i + n); };
        for (size_t k = 0; have(k + 1) && k < 7; ++k)
            if (T(k).results.empty() || T(k).reads.empty()) return 0;
        // softmax: max = ReduceMax(x); s = Sub(x, max); e = Exp(s); z = ReduceSum(e); y = Div(e, z)
        if (have(5) && T(0).type == "ReduceMax" && T(1).type == "Sub" && T(2).type == "Exp" && T(3).type == "ReduceSum" &&
            T(4).type == "Div" && last_axis(T(0)) && last_axis(T(3))) {
            const TensorDesc &x = T(0).reads[0], &y = res(4);
            if (reads_ids(T(1), x.id, res(0).id) && reads_ids(T(2), res(1).id) && reads_ids(T(3), res(2).id) &&
                reads_ids(T(4), res(2).id, res(3).id) && fp_type(x.dtype) && y.dtype == x.dtype && y.shape4() == x.shape4()) {
                auto ch = chain_of(5);
                bool ok = true;
                for (size_t k = 0; k < 4; ++k) ok = ok && private_to(res(k), ch, y.buffer_id);
                if (ok) {
                    fused = OpDesc();
                    fused.type = "Softmax";
                    fused.name = T(0).name + "..." + T(4).name;
                    fused.reads = {x};
                    fused.results = {y};
                    return 5;
                }
            }
        }
        // layernorm: m = ReduceMean(x); c = Sub(x, m); q = Mul(c, c); v = ReduceMean(q); a = ScalarAdd(v, eps);
        //            r = Rsqrt(a); y = Mul(c, r)
        if (have(7) && T(0).type == "ReduceMean" && T(1).type == "Sub" && T(2).type == "Mul" && T(3).type == "ReduceMean" &&
            T(4).type == "ScalarAdd" && T(5).type == "Rsqrt" && T(6).type == "Mul" && last_axis(T(0)) && last_axis(T(3))) {
            const TensorDesc &x = T(0).reads[0], &y = res(6);
            if (reads_ids(T(1), x.id, res(0).id) && reads_ids(T(2), res(1).id, res(1).id) && reads_ids(T(3), res(2).id) &&
                reads_ids(T(4), res(3).id) && reads_ids(T(5), res(4).id) && reads_ids(T(6), res(1).id, res(5).id) &&
                fp_type(x.dtype) && y.dtype == x.dtype && y.shape4() == x.shape4()) {
                auto ch = chain_of(7);
                bool ok = true;
                for (size_t k = 0; k < 6; ++k) ok = ok && private_to(res(k), ch, y.buffer_id);
                if (ok) {
                    fused = OpDesc();
                    fused.type = "LayerNorm";
                    fused.name = T(0).name + "..." + T(6).name;
                    fused.reads = {x};
                    fused.results = {y};
                    {
                        char eps[64];
                        snprintf(eps, sizeof(eps), "%.9g", T(4).arg_float("Factor"));
                        fused.args = Json::parse(std::string("{\"Eps\": {\"FLOAT\": ") + eps + "}}");
                    }
                    return 7;
                }
            }
        }
        // rmsnorm as the llama example writes it: f = Cast(x, fp32); q = Mul(f, f); m = ReduceMean(q); r = Rsqrt(m);
        // n = Mul(f, r); w = Mul(n, weight); y = Cast(w, type of x). No epsilon is added (examples/llama/model.py:96).
        if (have(7) && T(0).type == "Cast" && T(1).type == "Mul" && T(2).type == "ReduceMean" && T(3).type == "Rsqrt" &&
            T(4).type == "Mul" && T(5).type == "Mul" && T(6).type == "Cast" && last_axis(T(2))) {
            const TensorDesc &x = T(0).reads[0], &y = res(6);
            if (res(0).dtype == DT_F32 && (x.dtype == DT_F16 || x.dtype == DT_BF16) && y.dtype == x.dtype && y.shape4() == x.shape4() &&
                reads_ids(T(1), res(0).id, res(0).id) && reads_ids(T(2), res(1).id) && reads_ids(T(3), res(2).id) &&
                reads_ids(T(4), res(0).id, res(3).id) && T(5).reads.size() == 2 && T(5).reads[0].id == res(4).id &&
                reads_ids(T(6), res(5).id)) {
                const TensorDesc &w = T(5).reads[1];
                auto ch = chain_of(7);
                bool ok = w.dtype == DT_F32 && w.nelems() == x.shape4()[3] && w.dense();
                for (size_t k = 0; k < 6; ++k) ok = ok && private_to(res(k), ch, y.buffer_id);
                if (ok) {
                    fused = OpDesc();
                    fused.type = "RMSNorm";
                    fused.name = T(0).name + "..." + T(6).name;
                    fused.reads = {x, w};
                    fused.results = {y};
                    fused.args = Json::parse("{\"Eps\": {\"FLOAT\": 0.0}}");
                    return 7;
                }
            }
        }
        return 0;
    }

    // ---- task dispatch --------------------------------------------------------------------
    void lower_op(const OpDesc &op, const Range &proc, const TaskGroup &tg) {
        if (op.is_virtual) return;
        const std::string &t = op.type;
        if (t == "Noop" || t == "SendDone" || t == "Tensor" || t == "Refer" || t == "Reshape" || t == "Identity") return;
        if (t == "Rope" && rope_feeds_next_attention(op)) {  // the last operator of its task: nothing of this group follows it
            rope_for_attention = &op;
            return;
        }
        if (ewise_code(t) >= 0) return lower_ewise(op, proc, tg);
        if (t == "ReduceSum" || t == "ReduceMax" || t == "ReduceMean") return lower_reduce(op, proc, tg);
        if (t == "Matmul") return lower_matmul(op, proc, tg, -1, nullptr);
        if (t == "Transpose") return lower_transpose(op, proc, tg);
        if (t == "Embedding") return lower_embedding(op, proc, tg);
        if (t == "DecodeAttention") return lower_decode_attention(op, proc);
        if (t == "PrefillAttention") return lower_prefill_attention(op, proc);
        if (t == "RMSNorm" || t == "LayerNorm" || t == "Softmax") return lower_rowop(op, proc, &tg);
        if (t == "Send") return lower_send(op, proc);
        if (t == "Recv") return lower_recv(op, proc);
        if (t == "DeviceSync") return lower_device_sync(op, proc);
        if (t == "AllReduce") return lower_all_reduce(op, proc);
        if (t == "SendPacket") return lower_send_packet(op, proc, tg);
        if (t == "RecvPacket") return lower_recv_packet(op, proc, tg);
        if (t == "RecvReduceSendPacket") return lower_recv_reduce_send(op, proc, tg, true);
        if (t == "RecvReduceSend") return lower_recv_reduce_send(op, proc, tg, false);
        throw Error(E_UNSUPPORTED, "operator type not supported by this engine: " + t);
    }

    void lower_task_group(const TaskGroup &tg, const Range &proc) {
        const TaskInfo &ti = plan.task(tg.task_id);
        if (tg.task_range.count() == 0) return;
        bool first = true;
        for (size_t i = 0; i < ti.ops.size(); ++i) {
            const OpDesc &op = ti.ops[i];
            if (op.is_virtual) continue;
            {   // a softmax / layernorm / rmsnorm chain inside one task (the ops were merged with Sync=false)
                std::vector<const OpDesc *> seq;
                for (size_t j = i; j < ti.ops.size() && j < i + 7 && !ti.ops[j].is_virtual; ++j) seq.push_back(&ti.ops[j]);
                OpDesc fused;
                if (const size_t n = match_chain(seq, 0, fused)) {
                    if (!first) emit_sync(proc);
                    lower_rowop(fused, proc);
                    first = false;
                    i += n - 1;
                    continue;
                }
            }
            // Matmul followed by a unary activation on its result, merged into one task
            // by the planner (Sync=false): run the activation in the GEMM epilogue.
            // [RMSNorm | Mul] Matmul [activation] [Add]: one weight-streaming stage when the Matmul is one
            {
                GemvFuse gf;
                size_t mm = i;
                auto sole_input_of = [&](const OpDesc &prod, const OpDesc &cons) {
                    return !prod.results.empty() && !cons.reads.empty() && cons.reads[0].id == prod.results[0].id &&
                           other_readers(prod.results[0].buffer_id, &cons) == 0;
                };
                if (i + 1 < ti.ops.size() && ti.ops[i + 1].type == "Matmul" && sole_input_of(op, ti.ops[i + 1]) &&
                    matmul_is_gemv(ti.ops[i + 1], tg)) {
                    const TensorDesc &mx = ti.ops[i + 1].reads[0];
                    if (op.type == "RMSNorm" && op.reads[0].shape4() == mx.shape4() && op.reads[0].dtype == mx.dtype) {
                        const bool res = op.has_arg("Residual") && op.arg_bool("Residual");
                        size_t ri = 1;
                        gf.pro = GP_RMSNORM;
                        gf.x = &op.reads[0];
                        if (op.reads.size() > ri && op.reads[ri].nelems() == mx.shape4()[3]) gf.pro_a = &op.reads[ri++];
                        if (res && op.reads.size() > ri && op.results.size() >= 2) {
                            gf.pro_b = &op.reads[ri];
                            gf.pro_out = &op.results[1];
                        }
                        gf.eps = op.has_arg("Eps") ? (float)op.arg_float("Eps") : 1e-5f;
                        if (!res || gf.pro_b) mm = i + 1;
                    } else if (op.type == "Mul" && op.reads.size() == 2 && op.reads[0].shape4() == mx.shape4() &&
                               op.reads[1].shape4() == mx.shape4() && op.reads[0].dtype == mx.dtype && op.reads[1].dtype == mx.dtype) {
                        gf.pro = GP_MUL;
                        gf.x = &op.reads[0];
                        gf.pro_a = &op.reads[1];
                        mm = i + 1;
                    }
                    if (mm == i) gf = GemvFuse();
                }
                if (ti.ops[mm].type == "Matmul" && matmul_is_gemv(ti.ops[mm], tg)) {
                    const OpDesc &m = ti.ops[mm];
                    size_t last = mm;
                    int act = -1;
                    const TensorDesc *res_out = nullptr;
                    if (last + 1 < ti.ops.size()) {
                        const OpDesc &nx = ti.ops[last + 1];
                        const int ac = act_code(nx.type);
                        if (ac > 0 && nx.reads.size() == 1 && sole_input_of(m, nx) && nx.reads[0].shape == nx.results.at(0).shape &&
                            nx.results[0].dtype == m.results[0].dtype) {
                            act = ac;
                            res_out = &nx.results[0];
                            ++last;
                        }
                    }
                    if (act < 0 && last + 1 < ti.ops.size()) {
                        const OpDesc &nx = ti.ops[last + 1];
                        if (nx.type == "Add" && nx.reads.size() == 2 && !nx.results.empty() && nx.results[0].dtype == m.results[0].dtype &&
                            nx.reads[0].shape4() == m.results[0].shape4() && nx.reads[1].shape4() == m.results[0].shape4() &&
                            nx.results[0].shape4() == m.results[0].shape4() && other_readers(m.results[0].buffer_id, &nx) == 0) {
                            const bool first_is_mm = nx.reads[0].id == m.results[0].id, second_is_mm = nx.reads[1].id == m.results[0].id;
                            if (first_is_mm != second_is_mm) {
                                gf.residual = first_is_mm ? &nx.reads[1] : &nx.reads[0];
                                res_out = &nx.results[0];
                                ++last;
                            }
                        }
                    }
                    // Matmul -> one-shot AllReduce of its result (in place): the matmul stores into the staging slots itself
                    const OpDesc *ar = nullptr;
                    if (act < 0 && !gf.residual && last + 1 < ti.ops.size()) {
                        const OpDesc &nx = ti.ops[last + 1];
                        if (all_reduce_is_one_shot(nx) && !nx.reads.empty() && nx.reads[0].id == m.results[0].id &&
                            nx.results[0].buffer_id == m.results[0].buffer_id) {
                            ar = &nx;
                            gf.push_ord = oneshot_ord;
                        }
                    }
                    if (gf.pro != GP_NONE || gf.residual || ar) {
                        if (!first) emit_sync(proc);
                        lower_matmul(m, proc, tg, act, res_out, nullptr, &gf);
                        first = false;
                        i = last;
                        if (ar) {
                            const OpDesc *add = add_after_all_reduce(ti, i + 1);
                            // push not folded (K was split, or the result has a row pitch): the push stage reads what the
                            // matmul / its sum stage wrote with another split over the CTAs, so it waits for all of them
                            if (!gemv_pushed) emit_sync(proc);
                            lower_all_reduce(*ar, proc, false, gemv_pushed, add);
                            i += add ? 2 : 1;
                        }
                        continue;
                    }
                }
            }
            if (op.type == "Matmul" && fused_allreduce(plan, ti, i)) {
                if (!first) emit_sync(proc);
                lower_matmul(op, proc, tg, -1, nullptr, &ti.ops[i + 1]);
                lower_all_reduce(ti.ops[i + 1], proc, true);
                first = false;
                ++i;
                continue;
            }
            if (op.type == "Matmul" && !op.results.empty() && op.results[0].shape.size() == 2) {
                // Matmul [rows, heads * d] -> (reshape to [b, seq, heads, d]) -> Rope with a table [1, seq, 1, d]: the
                // rotation is applied to the accumulator, the unrotated projection is never stored
                size_t j = i + 1;
                while (j < ti.ops.size() && (ti.ops[j].is_virtual || ti.ops[j].type == "Reshape" || ti.ops[j].type == "Identity")) ++j;
                const bool fold_ok = []() { const char *e = getenv("ARKB_FOLD_EPILOGUE"); return e ? atoi(e) != 0 : true; }();
                if (fold_ok && j < ti.ops.size() && ti.ops[j].type == "Rope" && ti.ops[j].reads.size() == 2 && !ti.ops[j].results.empty()) {
                    const OpDesc &rp = ti.ops[j];
                    const TensorDesc &mmr = op.results[0], &x = rp.reads[0], &tab = rp.reads[1], &out = rp.results[0];
                    auto xs = x.shape4(), ts = tab.shape4();
                    const int64_t rows = mmr.shape[0], cols = mmr.shape[1];
                    const bool shapes = x.buffer_id == mmr.buffer_id && x.dense() && mmr.dense() && out.dense() && tab.dense() &&
                                        out.shape4() == xs && x.nelems() == rows * cols && xs[2] * xs[3] == cols && xs[0] * xs[1] == rows &&
                                        ts[0] == 1 && ts[2] == 1 && ts[1] == xs[1] && ts[3] == xs[3] && xs[3] % 8 == 0 &&
                                        tab.dtype == mmr.dtype && out.dtype == mmr.dtype && out.buffer_id != mmr.buffer_id;
                    int64_t org_x[4], o_x, org_m[4], o_m;
                    x.elem_strides(org_x, o_x);
                    mmr.elem_strides(org_m, o_m);
                    if (shapes && o_x == o_m && other_readers(mmr.buffer_id, &rp) == 0) {
                        TensorDesc view = out;  // the rope's result seen as the matmul's [rows, cols] output
                        view.shape = {rows, cols};
                        view.strides = {rows, cols};
                        view.offsets = {0, 0};
                        view.padded = {rows, cols};
                        if (out.offsets4() == std::vector<int64_t>{0, 0, 0, 0} && aligned16(tensor_ptr(tab)) &&
                            matmul_takes_epilogue_operand(op, tg, view, view)) {
                            if (!first) emit_sync(proc);
                            lower_matmul(op, proc, tg, -1, &view, nullptr, nullptr, &tab, 2, ts[1], ts[3]);
                            first = false;
                            i = j;
                            continue;
                        }
                    }
                }
            }
            if (op.type == "Matmul" && i + 1 < ti.ops.size() && (ti.ops[i + 1].type == "Add" || ti.ops[i + 1].type == "Mul")) {
                // Matmul -> Add / Mul with a tensor of the result's layout, the product having no other reader: the
                // tensor is read in the epilogue (residual add; gate * up of a SwiGLU block) and the product is never stored
                const OpDesc &nx = ti.ops[i + 1];
                if (nx.reads.size() == 2 && !nx.results.empty() && !op.results.empty()) {
                    const bool first_is_mm = nx.reads[0].id == op.results[0].id, second_is_mm = nx.reads[1].id == op.results[0].id;
                    const bool fold_ok = []() { const char *e = getenv("ARKB_FOLD_EPILOGUE"); return e ? atoi(e) != 0 : true; }();
                    if (fold_ok && first_is_mm != second_is_mm && other_readers(op.results[0].buffer_id, &nx) == 0) {
                        const TensorDesc &other = first_is_mm ? nx.reads[1] : nx.reads[0];
                        if (other.buffer_id != op.results[0].buffer_id && matmul_takes_epilogue_operand(op, tg, other, nx.results[0])) {
                            if (!first) emit_sync(proc);
                            lower_matmul(op, proc, tg, -1, &nx.results[0], nullptr, nullptr, &other, nx.type == "Mul" ? 1 : 0);
                            first = false;
                            ++i;
                            continue;
                        }
                    }
                }
            }
            if (op.type == "Matmul" && i + 1 < ti.ops.size()) {
                const OpDesc &nx = ti.ops[i + 1];
                const int act = act_code(nx.type);
                if (act > 0 && nx.reads.size() == 1 && nx.reads[0].id == op.results.at(0).id &&
                    nx.reads[0].shape == nx.results.at(0).shape && nx.results[0].dtype == op.results[0].dtype &&
                    (other_readers(op.results[0].buffer_id, &nx) == 0 || nx.results[0].buffer_id == op.results[0].buffer_id)) {
                    if (!first) emit_sync(proc);
                    lower_matmul(op, proc, tg, act, &nx.results[0]);
                    first = false;
                    ++i;
                    continue;
                }
            }
            if (op.type == "AllReduce") {
                if (const OpDesc *add = add_after_all_reduce(ti, i)) {
                    if (!first) emit_sync(proc);
                    lower_all_reduce(op, proc, false, false, add);
                    first = false;
                    ++i;
                    continue;
                }
            }
            const size_t before = prog.stages.size();
            if (!first) emit_sync(proc);  // ops of one task depend on each other; the split over CTAs differs per op
            const size_t mid = prog.stages.size();
            lower_op(op, proc, tg);
            if (prog.stages.size() == mid && mid != before) {  // op lowered to nothing: drop the barrier again
                const Stage &sy = prog.stages.back();
                --prog.syncs_per_iter[sy.sync_group];
                prog.stages.pop_back();
                prog.access.pop_back();
                prog.notes.pop_back();
            } else if (prog.stages.size() != mid) {
                first = false;
            }
        }
    }

    // CTA pairs (clusters of 2) can share matmul tiles when the grid is even and every
    // Matmul runs on a processor range made of whole pairs, over its full task range
    // (or with plan tiles that are multiples of 256 rows).
    bool pair_eligible() const {
        if (plan.num_processors % 2) return false;
        bool any = false;
        int64_t max_rows = 0;  // pairs share 256-row tiles: with at most 128 rows everywhere half of every pair would idle
        for (auto &pg : plan.processor_groups)
            for (auto &rg : pg.resource_groups)
                for (auto &tg : rg.task_groups)
                    for (auto &op : plan.task(tg.task_id).ops) {
                        if (op.type == "PrefillAttention") return false;  // its MMAs are issued per CTA (cta_group::1)
                        if (op.type != "Matmul") continue;
                        any = true;
                        if (!op.reads.empty() && !op.results.empty()) {
                            auto csh = op.results[0].shape4();
                            max_rows = std::max(max_rows, csh[2]);
                        }
                        if (rg.proc.s != 1 || rg.proc.b % 2 || rg.proc.count() % 2) return false;
                        if (!full_range(tg.task_range, num_tasks(op))) {
                            if (!op.config.is_object() || !op.config.contains("TileShapeMNK")) return false;
                            auto tile = op.config.at("TileShapeMNK").as_int_vec();
                            if (tile.size() != 3 || tile[0] % 256 || tile[1] % 32) return false;
                        }
                    }
        return any && max_rows > 128;
    }

    static void touched(const TaskInfo &ti, std::set<int64_t> &reads, std::set<int64_t> &writes) {
        for (auto &op : ti.ops) {
            for (auto &t : op.reads) reads.insert(t.buffer_id);
            for (auto &t : op.writes) writes.insert(t.buffer_id);
            for (auto &t : op.results) writes.insert(t.buffer_id);
        }
    }

    // ---- barriers no dependency needs -----------------------------------------------------------------
    static bool overlap(const std::pair<uintptr_t, uintptr_t> &a, const std::pair<uintptr_t, uintptr_t> &b) {
        return a.first < b.second && b.first < a.second;
    }
    // Does stage y have to see (or must it not disturb) what stage x did? Two flat elementwise walks over the same
    // CTAs with the same unit count and size touch a common operand thread by thread, so an operand both start at
    // the same address orders itself by program order inside each thread.
    bool depends(size_t xi, size_t yi) const {
        const StageAccess &x = prog.access[xi], &y = prog.access[yi];
        if (x.opaque || y.opaque) return true;
        const Stage &sx = prog.stages[xi], &sy = prog.stages[yi];
        const bool aligned = x.aligned_units > 0 && x.aligned_units == y.aligned_units && x.aligned_unit_bytes == y.aligned_unit_bytes &&
                             sx.proc_b == sy.proc_b && sx.proc_e == sy.proc_e && sx.proc_s == sy.proc_s;
        const bool same_tiles = x.tile_sig != 0 && x.tile_sig == y.tile_sig && sx.proc_b == sy.proc_b && sx.proc_e == sy.proc_e &&
                                sx.proc_s == sy.proc_s;
        auto in = [](const std::vector<std::pair<uintptr_t, uintptr_t>> &v, const std::pair<uintptr_t, uintptr_t> &a) {
            for (auto &e : v) if (e == a) return true;
            return false;
        };
        auto hit = [&](const std::pair<uintptr_t, uintptr_t> &a, const std::pair<uintptr_t, uintptr_t> &b) {
            if (!overlap(a, b)) return false;
            if (aligned && a.first == b.first) return false;
            // a matmul's output tile read back as the epilogue operand of a matmul with the same tiles: same CTA
            if (same_tiles && a == b && in(x.tiled, a) && in(y.tiled, b)) return false;
            return true;
        };
        for (auto &w : x.writes) {
            for (auto &r : y.reads) if (hit(w, r)) return true;
            for (auto &v : y.writes) if (hit(w, v)) return true;
        }
        for (auto &r : x.reads)
            for (auto &v : y.writes) if (hit(r, v)) return true;
        return false;
    }

    // The straightforward lowering puts a barrier wherever the plan's rules or the op order might need one. This
    // pass keeps a barrier only when a stage behind it (up to the next barrier) depends on a stage that ran since
    // the last whole-grid barrier that was kept; the barrier at the end of every iteration closes the rest.
    void elide_syncs() {
        if (const char *e = getenv("ARKB_KEEP_SYNCS")) if (atoi(e)) return;
        const size_t n = prog.stages.size();
        std::vector<bool> keep(n, true);
        std::vector<size_t> pending;
        for (size_t i = 0; i < n; ++i) {
            const Stage &s = prog.stages[i];
            if (s.kind == SK_PEERSYNC && s.ps.with_grid) {  // a barrier that is never elided
                if (s.proc_b == 0 && s.proc_s == 1 && s.proc_e >= prog.grid) pending.clear();
                else pending.push_back(i);
                continue;
            }
            if (s.kind != SK_SYNC) {
                pending.push_back(i);
                continue;
            }
            bool needed = false;
            auto whole_grid_barrier = [&](const Stage &b) {
                return b.kind == SK_PEERSYNC && b.ps.with_grid && b.proc_b == 0 && b.proc_s == 1 && b.proc_e >= prog.grid;
            };
            for (size_t j = i + 1; j < n && prog.stages[j].kind != SK_SYNC && !whole_grid_barrier(prog.stages[j]) && !needed; ++j)
                for (size_t x : pending)
                    if (depends(x, j)) { needed = true; break; }
            if (!needed) {
                keep[i] = false;
                continue;
            }
            if (s.proc_b == 0 && s.proc_s == 1 && s.proc_e >= prog.grid) pending.clear();
        }
        Program out = prog;
        out.stages.clear(); out.access.clear(); out.notes.clear();
        for (int g = 0; g < kMaxSyncGroups; ++g) out.syncs_per_iter[g] = 0;
        for (size_t i = 0; i < n; ++i) {
            if (!keep[i]) { ++out.syncs_elided; continue; }
            Stage s = prog.stages[i];
            std::string note = prog.notes[i];
            if (s.kind == SK_PEERSYNC && s.ps.with_grid) s.sync_ord = ++out.syncs_per_iter[s.sync_group];
            if (s.kind == SK_SYNC) {
                s.sync_ord = ++out.syncs_per_iter[s.sync_group];
                const size_t at = note.find("sync group");
                note = note.substr(0, at) + "sync group " + std::to_string(s.sync_group) + " #" + std::to_string(s.sync_ord);
            }
            out.stages.push_back(s);
            out.access.push_back(prog.access[i]);
            out.notes.push_back(note);
        }
        prog = out;
    }

    // Two weight-streaming matmuls that follow each other without a barrier, over the same activations with the same
    // prologue and of the same shape (W1 and W3 of a SwiGLU block), become one stage: x is normalised and staged once,
    // and the CTAs' row shares are cut from both matrices together, so that the pipeline ramps up and drains once.
    void pair_weight_streams() {
        if (const char *e = getenv("ARKB_PAIR_GEMV")) if (!atoi(e)) return;
        for (size_t i = 0; i + 1 < prog.stages.size(); ++i) {
            Stage &s0 = prog.stages[i];
            const Stage &s1 = prog.stages[i + 1];
            if (s0.kind != SK_GEMV || s1.kind != SK_GEMV) continue;
            GemvArgs &a = s0.gv;
            const GemvArgs &b = s1.gv;
            if (s0.proc_b != s1.proc_b || s0.proc_e != s1.proc_e || s0.proc_s != s1.proc_s) continue;
            if (!a.w_is_nk || !b.w_is_nk || a.w_b || b.w_b || a.splits != 1 || b.splits != 1) continue;
            if (a.x != b.x || a.pro != b.pro || a.pro_a != b.pro_a || a.pro_b != b.pro_b || a.src_ord != b.src_ord || a.pro_eps != b.pro_eps ||
                a.pro == GP_ATTN_MERGE)
                continue;
            if (a.M != b.M || a.N != b.N || a.K != b.K || a.ldx != b.ldx || a.ldw != b.ldw || a.ldo != b.ldo || a.dtype != b.dtype ||
                a.rows_together != b.rows_together || a.light != b.light || a.kper != b.kper || a.ctas_per_split != b.ctas_per_split)
                continue;
            if (a.residual || b.residual || a.push_ord || b.push_ord || b.pro_out) continue;
            a.w_b = b.w;
            a.out_b = b.out;
            a.act_b = b.act;
            {   // rows a warp walks together, for twice the rows (the time model of lower_matmul, one k-range)
                const int64_t warps = kThreads / 32, loads = (a.M == 1 ? 8 : 4) / (a.light ? 2 : 1);
                const int64_t rows_cta = (2 * (int64_t)a.N + a.ctas_per_split - 1) / a.ctas_per_split;
                double best = 1e30;
                for (int64_t RW = loads; RW >= 1; RW /= 2) {
                    const int64_t VC = loads / RW;
                    const int64_t rounds = ((rows_cta + RW - 1) / RW + warps - 1) / warps;
                    const double steps = (double)((a.kper + 256 * VC - 1) / (256 * VC));
                    const double t = (double)rounds * (steps + 1.5) * (1.0 + 0.03 * (double)(VC - 1));
                    if (t < best - 1e-9) { best = t; a.rows_together = (int32_t)RW; }
                }
            }
            // the stage touches what both touched
            StageAccess &x = prog.access[i];
            const StageAccess &y = prog.access[i + 1];
            x.reads.insert(x.reads.end(), y.reads.begin(), y.reads.end());
            x.writes.insert(x.writes.end(), y.writes.begin(), y.writes.end());
            x.streamed.insert(x.streamed.end(), y.streamed.begin(), y.streamed.end());
            x.opaque = x.opaque || y.opaque;
            prog.notes[i] += "  + " + prog.notes[i + 1].substr(prog.notes[i + 1].find("Matmul(gemv) ") + 13, prog.notes[i + 1].find(" M=") - prog.notes[i + 1].find("Matmul(gemv) ") - 13) +
                             " (second matrix, act=" + std::to_string(b.act) + ", rows/warp-step=" + std::to_string(a.rows_together) + ")";
            prog.stages.erase(prog.stages.begin() + i + 1);
            prog.access.erase(prog.access.begin() + i + 1);
            prog.notes.erase(prog.notes.begin() + i + 1);
        }
    }

    // Barriers fetch ahead: operands that no op of the plan writes (weights, K/V caches) are asked into L2 by the
    // barrier stages that precede their readers, as early as a budget of bytes in flight allows, so that a chain of
    // small dependent stages (decode) waits on L2 hits instead of HBM round trips, and HBM streams while CTAs sit
    // at barriers. The stage list is cyclic: the last barriers of an iteration fetch for the first stages of the next.
    void plan_prefetch() {
        if (const char *e = getenv("ARKB_PREFETCH")) if (!atoi(e)) return;
        const size_t n = prog.stages.size();
        std::set<int64_t> written;
        for (auto &ti : plan.task_infos)
            for (auto &op : ti.ops) {
                for (auto &t : op.writes) written.insert(t.buffer_id);
                for (auto &t : op.results) written.insert(t.buffer_id);
            }
        struct Item { size_t stage; const void *ptr; size_t bytes; };
        std::vector<Item> items;
        for (size_t i = 0; i < n; ++i)
            for (auto &sd : prog.access[i].streamed)
                if (!written.count(sd.buffer_id)) items.push_back({i, sd.ptr, sd.bytes});
        std::vector<size_t> syncs;
        for (size_t i = 0; i < n; ++i)  // barriers of at least 32 CTAs: each CTA asks for its share
            if (prog.stages[i].kind == SK_SYNC && prog.stages[i].sync_count >= 32) syncs.push_back(i);
        if (items.empty() || syncs.empty()) return;
        size_t kBudget = 16u << 20;  // bytes fetched but not yet read: more than this ahead cost time (measured on decode)
        if (const char *e = getenv("ARKB_PREFETCH_MB")) kBudget = (size_t)std::max(1, atoi(e)) << 20;
        // walk the cyclic schedule twice: the first lap only warms up the window, the second lap's choices are kept
        size_t next = 0, outstanding = 0;
        std::vector<std::pair<size_t, size_t>> inflight;  // (absolute consumer position, bytes)
        const size_t ni = items.size();
        auto abs_pos = [&](size_t lap, size_t stage) { return lap * n + stage; };
        // items are consumed in order; `next` counts items assigned so far over both laps
        for (size_t lap = 0; lap < 2; ++lap)
            for (size_t si = 0; si < syncs.size(); ++si) {
                const size_t here = abs_pos(lap, syncs[si]);
                for (auto it = inflight.begin(); it != inflight.end();)
                    if (it->first < here) { outstanding -= it->second; it = inflight.erase(it); } else ++it;
                Stage &sy = prog.stages[syncs[si]];
                if (lap == 1) sy.sy.n_pf = 0;
                while (true) {
                    const Item &itx = items[next % ni];
                    size_t cons = abs_pos(next / ni, itx.stage);
                    while (cons < here) { ++next; cons = abs_pos(next / ni, items[next % ni].stage); }
                    const Item &it = items[next % ni];
                    if (cons > here + n) break;                      // never more than one lap ahead
                    if (outstanding > 0 && outstanding + it.bytes > kBudget) break;
                    const size_t bytes = std::min(it.bytes, kBudget);  // a huge operand: its head only
                    if (lap == 1) {
                        if (sy.sy.n_pf >= kMaxPrefetch) break;
                        sy.sy.pf_ptr[sy.sy.n_pf] = it.ptr;
                        sy.sy.pf_bytes[sy.sy.n_pf] = bytes;
                        ++sy.sy.n_pf;
                        prog.prefetch_bytes += bytes;
                    }
                    inflight.push_back({cons, bytes});
                    outstanding += bytes;
                    ++next;
                }
            }
        for (size_t i : syncs)
            if (prog.stages[i].sy.n_pf > 0) {
                size_t b = 0;
                for (int k = 0; k < prog.stages[i].sy.n_pf; ++k) b += prog.stages[i].sy.pf_bytes[k];
                prog.notes[i] += " +L2 prefetch " + std::to_string(b >> 10) + " KiB";
            }
    }

    void run() {
        if (plan.num_processors > env.num_sm)
            throw Error(E_UNSUPPORTED, "plan needs " + std::to_string(plan.num_processors) + " processors, the device has " +
                                           std::to_string(env.num_sm) + " SMs (the loop kernel keeps one CTA per processor resident)");
        prog.grid = plan.num_processors;
        prog.pair_mode = env.allow_pair && pair_eligible();
        std::vector<Range> unsynced;
        bool first_pg = true;
        // a processor group that holds exactly one operator over its full task range: the only op of the only task of
        // its only resource group (what the planner emits for an operator outside any context)
        auto single_op = [&](const ProcessorGroup &g) -> const OpDesc * {
            if (g.resource_groups.size() != 1 || g.resource_groups[0].task_groups.size() != 1) return nullptr;
            const TaskGroup &tg = g.resource_groups[0].task_groups[0];
            const TaskInfo &ti = plan.task(tg.task_id);
            const OpDesc *only = nullptr;
            for (auto &o : ti.ops) {
                if (o.is_virtual) continue;
                if (only) return nullptr;
                only = &o;
            }
            if (!only || !full_range(tg.task_range, num_tasks(*only))) return nullptr;
            return only;
        };
        size_t skip_pgs = 0;
        for (size_t pgi = 0; pgi < plan.processor_groups.size(); ++pgi) {
            if (skip_pgs) { --skip_pgs; continue; }
            cur_pg = pgi;
            if (pending_sum.buffer_id >= 0 && !sum_consumer(pgi, pending_sum.buffer_id, pending_sum.rows, pending_sum.cols)) {
                if (!pending_sum.stored) throw Error(E_INTERNAL, "one-shot all_reduce sum was left without a consumer");
                pending_sum = PendingSum();
            }
            const ProcessorGroup *pgp = &plan.processor_groups[pgi];
            if (const OpDesc *o = single_op(*pgp)) {
                if (rope_feeds_next_attention(*o)) {
                    rope_for_attention = o;
                    continue;
                }
            }
            ProcessorGroup merged;
            {   // a chain spread over consecutive single-operator processor groups becomes one group with one fused operator
                std::vector<const OpDesc *> seq;
                Range widest = pgp->proc;
                for (size_t k = pgi; k < plan.processor_groups.size() && k < pgi + 7; ++k) {
                    const OpDesc *o = single_op(plan.processor_groups[k]);
                    if (!o) break;
                    seq.push_back(o);
                }
                OpDesc fused;
                if (const size_t n = seq.empty() ? 0 : match_chain(seq, 0, fused)) {
                    for (size_t k = pgi; k < pgi + n; ++k) {
                        const Range &r = plan.processor_groups[k].proc;
                        if (r.s == 1 && r.count() > widest.count()) widest = r;
                    }
                    fused_ops.push_back(fused);
                    merged.proc = widest;
                    chain_pgs[pgi] = fused_ops.size() - 1;
                    skip_pgs = n - 1;
                }
            }
            const ProcessorGroup &pg = chain_pgs.count(pgi) ? merged : *pgp;
            const Range &pr = pg.proc;
            if (pr.count() == 0) continue;
            if (!first_pg) {
                // barrier rule of the reference code generator (ark/codegen.cpp:109-158)
                bool need_sync = false;
                for (auto it = unsynced.begin(); it != unsynced.end();) {
                    if (!pr.overlaps(*it)) {
                        ++it;
                        continue;
                    }
                    const bool range_inside_pr = it->b >= pr.b && it->e <= pr.e && pr.s == 1;
                    if (!range_inside_pr) {
                        emit_sync(*it);
                        const bool pr_inside_range = pr.b >= it->b && pr.e <= it->e && it->s == 1;
                        if (!pr_inside_range) need_sync = true;
                    } else {
                        need_sync = true;
                    }
                    it = unsynced.erase(it);
                }
                if (need_sync) emit_sync(pr);
            }
            if (chain_pgs.count(pgi)) lower_rowop(fused_ops[chain_pgs[pgi]], pr);
            for (auto &rg : pg.resource_groups) {
                std::set<int64_t> prev_w;
                bool any = false;
                for (auto &tg : rg.task_groups) {
                    std::set<int64_t> r, w;
                    touched(plan.task(tg.task_id), r, w);
                    bool conflict = false;
                    for (auto b : prev_w)
                        if (r.count(b) || w.count(b)) conflict = true;
                    // The reference runs task groups of one resource group back to back on each
                    // processor with no barrier, relying on its task->processor mapping. This
                    // engine splits work differently, so dependent groups get a barrier.
                    if (any && conflict) emit_sync(rg.proc);
                    lower_task_group(tg, rg.proc);
                    prev_w.insert(w.begin(), w.end());
                    any = true;
                }
            }
            unsynced.push_back(pr);
            first_pg = false;
            if (pending_merge.buffer_id >= 0 && pending_merge_pg != pgi)
                throw Error(E_INTERNAL, "decode attention merge was left without its consumer");
        }
        if (pending_merge.buffer_id >= 0) throw Error(E_INTERNAL, "decode attention merge was left without its consumer");
        if (pending_sum.buffer_id >= 0 && !pending_sum.stored) throw Error(E_INTERNAL, "one-shot all_reduce sum was left without a consumer");
        elide_syncs();
        pair_weight_streams();
        plan_prefetch();
        // dynamic shared memory: the largest need of any stage
        size_t smem = 16 * 1024;
        for (auto &s : prog.stages) {
            size_t need = 0;
            switch (s.kind) {
                case SK_GEMM: need = kFullSmemBytes; break;
                case SK_PREFILL_ATTN: need = kFullSmemBytes; break;
                case SK_GEMM_SIMT: need = 16 * 1024; break;
                case SK_REDUCE: need = (size_t)kThreads * 8 * sizeof(float); break;
                case SK_ROWOP:
                    if (s.ro.staged_warps > 0) {
                        const size_t row = (size_t)s.ro.cols * dtype_size(s.ro.dtype);
                        const size_t wrow = s.ro.weight_smem ? (size_t)s.ro.cols * (s.ro.weight_f32 ? 4 : dtype_size(s.ro.dtype)) : 0;
                        need = (size_t)s.ro.staged_warps * s.ro.staged_bufs * ((row + 127) / 128 * 128) + (wrow + 127) / 128 * 128 + 1024;
                    } else {
                        need = 16 * 1024;
                    }
                    break;
                case SK_GEMV:
                    need = (size_t)s.gv.M * (size_t)std::max(s.gv.kper, s.gv.K) * sizeof(float) + 4096;
                    break;
                case SK_DECODE_ATTN: {
                    const size_t G = (size_t)(s.da.Hq / std::max(1, s.da.Hkv));
                    need = (G * 128 + 16 + G * (size_t)s.da.chunk_len + 16 * G * 128) * sizeof(float) + 1024;
                    break;
                }
                default: break;
            }
            smem = std::max(smem, need);
        }
        prog.smem_bytes = std::min<size_t>((smem + 1023) / 1024 * 1024, kFullSmemBytes);
        if (const char *e = getenv("ARKB_FULL_SMEM")) if (atoi(e)) prog.smem_bytes = kFullSmemBytes;
        prog.n_sync_groups = (int)sync_ids.size();
        prog.oneshots_per_iter = oneshot_ord;
        for (auto &s : prog.stages) {
            if (s.kind == SK_ALLREDUCE && s.ar.algo == 0) s.ar.per_iter = oneshot_ord;
            if (s.kind == SK_GEMV && (s.gv.push_ord > 0 || s.gv.src_ord > 0)) {
                s.gv.push_per_iter = oneshot_ord;
                s.gv.push_stage_bytes = lay.comm_stage_bytes;
            }
        }
    }
};

}  // namespace

std::string Program::dump() const {
    std::ostringstream os;
    os << "grid=" << grid << (pair_mode ? " pairs" : "") << " stages=" << stages.size() << " sync_groups=" << n_sync_groups
       << " peer_barriers=" << peersyncs_per_iter << (syncs_elided ? " barriers_elided=" + std::to_string(syncs_elided) : "") << "\n";
    for (size_t i = 0; i < notes.size(); ++i) os << i << ": " << notes[i] << "\n";
    return os.str();
}

Program lower_plan(const Plan &plan, const Layout &lay, const LowerEnv &env) {
    Lowerer lw(plan, lay, env);
    lw.run();
    return lw.prog;
}

}  // namespace arkb
