// Plan JSON -> host IR, and the arena layout.
#include "plan.hpp"

#include <algorithm>
#include <cstdlib>
#include <set>

namespace arkb {

int dtype_from_name(const std::string &n) {
    // names as serialised by the reference (ark/api/data_type.cpp:28-36)
    if (n == "FP32") return DT_F32;
    if (n == "FP16") return DT_F16;
    if (n == "BF16") return DT_BF16;
    if (n == "INT32") return DT_I32;
    if (n == "UINT32") return DT_U32;
    if (n == "INT8") return DT_I8;
    if (n == "UINT8" || n == "BYTE") return DT_U8;
    throw Error(E_MODEL, "unknown data type: " + n);
}

size_t dtype_size(int dt) {
    switch (dt) {
        case DT_F32: case DT_I32: case DT_U32: return 4;
        case DT_F16: case DT_BF16: return 2;
        default: return 1;
    }
}

static std::vector<int64_t> pad4(const std::vector<int64_t> &v, int64_t fill) {
    if (v.size() > 4) throw Error(E_MODEL, "tensors have at most 4 dimensions");
    std::vector<int64_t> r(4 - v.size(), fill);
    r.insert(r.end(), v.begin(), v.end());
    return r;
}

TensorDesc TensorDesc::from_json(const Json &j) {
    TensorDesc t;
    try {
        t.id = j.at("Id").as_int();
        t.dtype = dtype_from_name(j.at("DataType").as_string());
        t.shape = j.at("Shape").as_int_vec();
        t.strides = j.contains("Strides") ? j.at("Strides").as_int_vec() : t.shape;
        t.offsets = j.contains("Offsets") ? j.at("Offsets").as_int_vec() : std::vector<int64_t>(t.shape.size(), 0);
        t.padded = j.contains("PaddedShape") ? j.at("PaddedShape").as_int_vec() : t.shape;
        const Json &b = j.at("Buffer");
        t.buffer_id = b.at("Id").as_int();
        t.buffer_rank = b.contains("Rank") ? (int)b.at("Rank").as_int() : -1;
        auto tags = [](const Json &a, std::vector<std::pair<int, int>> &out) {
            for (auto &e : a.arr) out.emplace_back((int)e.at(0).as_int(), (int)e.at(1).as_int());
        };
        if (b.contains("SendTags")) tags(b.at("SendTags"), t.send_tags);
        if (b.contains("RecvTags")) tags(b.at("RecvTags"), t.recv_tags);
    } catch (const Error &) {
        throw;
    } catch (const std::exception &e) {
        throw Error(E_MODEL, std::string("bad tensor description: ") + e.what());
    }
    const size_t nd = t.shape.size();
    if (t.strides.size() != nd || t.offsets.size() != nd || t.padded.size() != nd)
        throw Error(E_MODEL, "tensor shape/strides/offsets/padded_shape rank mismatch");
    // invariants of ark/model/model_tensor.cpp:27-77
    for (size_t i = 0; i < nd; ++i) {
        if (t.shape[i] > t.padded[i] || t.offsets[i] + t.padded[i] > t.strides[i])
            throw Error(E_MODEL, "tensor " + std::to_string(t.id) + ": shape <= padded_shape and offsets + padded_shape <= strides must hold");
    }
    return t;
}

int64_t TensorDesc::nelems() const {
    int64_t n = 1;
    for (auto v : shape) n *= v;
    return n;
}
int64_t TensorDesc::stride_bytes() const {
    int64_t n = 1;
    for (auto v : strides) n *= v;
    return n * (int64_t)dtype_size(dtype);
}
std::vector<int64_t> TensorDesc::shape4() const { return pad4(shape, 1); }
std::vector<int64_t> TensorDesc::strides4() const { return pad4(strides, 1); }
std::vector<int64_t> TensorDesc::offsets4() const { return pad4(offsets, 0); }

void TensorDesc::elem_strides(int64_t (&es)[4], int64_t &origin) const {
    auto st = strides4();
    auto of = offsets4();
    es[3] = 1;
    es[2] = st[3];
    es[1] = st[2] * st[3];
    es[0] = st[1] * st[2] * st[3];
    origin = 0;
    for (int i = 0; i < 4; ++i) origin += of[i] * es[i];  // ark/model/model_offset.cpp:13-27
}

bool TensorDesc::dense() const {
    int64_t es[4], org;
    elem_strides(es, org);
    auto sh = shape4();
    int64_t expect = 1;
    for (int i = 3; i >= 0; --i) {
        if (sh[i] > 1 && es[i] != expect) return false;
        expect *= sh[i];
    }
    return true;
}

Range Range::from_json(const Json &j) {
    Range r;
    if (!j.is_array() || (j.size() != 2 && j.size() != 3)) throw Error(E_PLAN, "a range is [begin, end] or [begin, end, step]");
    r.b = j.at(0).as_int();
    r.e = j.at(1).as_int();
    r.s = j.size() == 3 ? j.at(2).as_int() : 1;
    if (r.s <= 0) throw Error(E_PLAN, "range step must be positive");
    return r;
}

bool Range::overlaps(const Range &o) const {
    if (count() == 0 || o.count() == 0) return false;
    if (e <= o.b || o.e <= b) return false;
    if (s == 1 && o.s == 1) return true;
    for (int64_t v = b; v < e; v += s) {
        if (v >= o.b && v < o.e && (v - o.b) % o.s == 0) return true;
    }
    return false;
}

int64_t OpDesc::arg_int(const std::string &k) const {
    const Json &a = args.at(k);
    if (!a.is_object() || a.obj.empty()) throw Error(E_MODEL, "bad argument " + k);
    return a.obj[0].second.as_int();
}
double OpDesc::arg_float(const std::string &k) const {
    const Json &a = args.at(k);
    if (!a.is_object() || a.obj.empty()) throw Error(E_MODEL, "bad argument " + k);
    return a.obj[0].second.as_float();
}
bool OpDesc::arg_bool(const std::string &k) const {
    const Json &a = args.at(k);
    if (!a.is_object() || a.obj.empty()) throw Error(E_MODEL, "bad argument " + k);
    return a.obj[0].second.as_bool();
}
std::vector<int64_t> OpDesc::arg_dims(const std::string &k) const {
    const Json &a = args.at(k);
    if (!a.is_object() || a.obj.empty()) throw Error(E_MODEL, "bad argument " + k);
    return a.obj[0].second.as_int_vec();
}

Plan Plan::parse(const std::string &text) {
    Json j;
    try {
        j = Json::parse(text);
    } catch (const std::exception &e) {
        throw Error(E_PLAN, std::string("plan is not valid JSON: ") + e.what());
    }
    Plan p;
    try {
        // required fields as validated by the reference (ark/model/model_json.cpp:259-284)
        for (const char *k : {"Rank", "WorldSize", "NumProcessors", "NumWarpsPerProcessor", "TaskInfos", "ProcessorGroups"})
            if (!j.contains(k)) throw Error(E_PLAN, std::string("plan lacks field ") + k);
        p.rank = (int)j.at("Rank").as_int();
        p.world_size = (int)j.at("WorldSize").as_int();
        p.architecture = j.contains("Architecture") ? j.at("Architecture").as_string() : "ANY";
        p.num_processors = (int)j.at("NumProcessors").as_int();
        p.num_warps_per_processor = (int)j.at("NumWarpsPerProcessor").as_int();
        p.arena_reuse = j.contains("ArenaReuse") ? j.at("ArenaReuse").as_bool() : false;
        if (const char *e = getenv("ARKB_ARENA_REUSE")) p.arena_reuse = atoi(e) != 0;
        if (p.rank < 0 || p.rank >= p.world_size) throw Error(E_USAGE, "rank " + std::to_string(p.rank) + " outside world size " + std::to_string(p.world_size));
        if (p.world_size > kMaxPeers) throw Error(E_UNSUPPORTED, "world size above " + std::to_string(kMaxPeers));
        if (p.num_processors < 1) throw Error(E_PLAN, "NumProcessors must be positive");
        for (auto &tj : j.at("TaskInfos").arr) {
            TaskInfo ti;
            ti.id = tj.at("Id").as_int();
            ti.num_warps = (int)tj.at("NumWarps").as_int();
            ti.sram_bytes = (int)tj.at("SramBytes").as_int();
            for (auto &oj : tj.at("Ops").arr) {
                OpDesc op;
                op.type = oj.at("Type").as_string();
                op.name = oj.contains("Name") ? oj.at("Name").as_string() : "";
                op.is_virtual = oj.contains("IsVirtual") ? oj.at("IsVirtual").as_bool() : false;
                for (auto &t : oj.at("ReadTensors").arr) op.reads.push_back(TensorDesc::from_json(t));
                for (auto &t : oj.at("WriteTensors").arr) op.writes.push_back(TensorDesc::from_json(t));
                for (auto &t : oj.at("ResultTensors").arr) op.results.push_back(TensorDesc::from_json(t));
                if (oj.contains("Args")) op.args = oj.at("Args");
                if (oj.contains("Config")) op.config = oj.at("Config");
                ti.ops.push_back(std::move(op));
            }
            p.task_infos.push_back(std::move(ti));
        }
        for (auto &pj : j.at("ProcessorGroups").arr) {
            ProcessorGroup pg;
            pg.proc = Range::from_json(pj.at("ProcessorRange"));
            for (auto &rj : pj.at("ResourceGroups").arr) {
                ResourceGroup rg;
                rg.proc = Range::from_json(rj.at("ProcessorRange"));
                rg.warp = Range::from_json(rj.at("WarpRange"));
                rg.sram = Range::from_json(rj.at("SramRange"));
                for (auto &gj : rj.at("TaskGroups").arr) {
                    TaskGroup tg;
                    tg.task_id = gj.at("TaskId").as_int();
                    tg.task_range = Range::from_json(gj.at("TaskRange"));
                    tg.granularity = gj.contains("Granularity") ? gj.at("Granularity").as_int() : 1;
                    if (tg.granularity < 1) throw Error(E_PLAN, "Granularity must be positive");
                    rg.task_groups.push_back(tg);
                }
                if (rg.proc.b < pg.proc.b || rg.proc.e > pg.proc.e)
                    throw Error(E_PLAN, "a resource group's ProcessorRange must lie inside its processor group's");
                pg.resource_groups.push_back(std::move(rg));
            }
            if (pg.proc.e > p.num_processors) throw Error(E_PLAN, "ProcessorRange exceeds NumProcessors");
            p.processor_groups.push_back(std::move(pg));
        }
    } catch (const Error &) {
        throw;
    } catch (const std::exception &e) {
        throw Error(E_PLAN, std::string("malformed plan: ") + e.what());
    }
    for (auto &pg : p.processor_groups)
        for (auto &rg : pg.resource_groups)
            for (auto &tg : rg.task_groups) p.task(tg.task_id);
    return p;
}

const TaskInfo &Plan::task(int64_t id) const {
    for (auto &t : task_infos)
        if (t.id == id) return t;
    throw Error(E_PLAN, "TaskGroup refers to unknown TaskId " + std::to_string(id));
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

bool fused_allreduce(const Plan &plan, const TaskInfo &ti, size_t i) {
    if (plan.world_size < 2 || plan.world_size > kMaxPeers || i + 1 >= ti.ops.size()) return false;
    const OpDesc &mm = ti.ops[i], &ar = ti.ops[i + 1];
    if (mm.type != "Matmul" || ar.type != "AllReduce" || mm.results.empty() || ar.results.empty() || ar.reads.empty()) return false;
    const TensorDesc &c = mm.results[0];
    if (ar.reads[0].id != c.id || ar.results[0].buffer_id != c.buffer_id) return false;
    if (c.dtype != DT_F16 && c.dtype != DT_BF16) return false;
    if (!c.dense()) return false;
    auto sh = c.shape4();
    if (sh[0] != 1 || sh[1] != 1) return false;
    return sh[2] % (256 * (int64_t)plan.world_size) == 0 && sh[3] % 32 == 0;
}

Layout plan_layout(const Plan &plan) {
    Layout lay;
    auto visit = [&](const TensorDesc &t) {
        auto it = lay.buffers.find(t.buffer_id);
        if (it == lay.buffers.end()) {
            BufferInfo bi;
            bi.id = t.buffer_id;
            bi.rank = t.buffer_rank;
            it = lay.buffers.emplace(t.buffer_id, bi).first;
        }
        BufferInfo &bi = it->second;
        bi.bytes = std::max(bi.bytes, (size_t)t.stride_bytes());
        for (auto &tg : t.send_tags)
            if (std::find(bi.send_tags.begin(), bi.send_tags.end(), tg) == bi.send_tags.end()) bi.send_tags.push_back(tg);
        for (auto &tg : t.recv_tags)
            if (std::find(bi.recv_tags.begin(), bi.recv_tags.end(), tg) == bi.recv_tags.end()) bi.recv_tags.push_back(tg);
    };
    size_t oneshot_max = 0;
    for (auto &ti : plan.task_infos)
        for (auto &op : ti.ops) {
            for (auto &t : op.reads) visit(t);
            for (auto &t : op.writes) visit(t);
            for (auto &t : op.results) visit(t);
            if (op.type == "AllReduce" && !op.results.empty())
                oneshot_max = std::max(oneshot_max, (size_t)op.results[0].nelems() * dtype_size(op.results[0].dtype));
        }
    // ---- lifetimes of intermediates (only when the plan asks for reuse) ----
    struct Life { int first = -1, last = -1; bool ok = true, written = false, read = false, first_is_write = false; };
    std::map<int64_t, Life> life;
    if (plan.arena_reuse) {
        auto whole = [&](const TensorDesc &t) {
            const BufferInfo &b = lay.buffers.at(t.buffer_id);
            for (auto o : t.offsets) if (o) return false;
            return t.dense() && t.shape == t.padded && (size_t)t.nelems() * dtype_size(t.dtype) == b.bytes;
        };
        static const std::set<std::string> comm_ops = {"Send", "SendDone", "Recv", "DeviceSync", "AllReduce", "SendPacket",
                                                        "RecvPacket", "RecvReduceSendPacket", "RecvReduceSend"};
        int step = 0;
        for (auto &pg : plan.processor_groups) {
            for (auto &rg : pg.resource_groups)
                for (auto &tg : rg.task_groups)
                    for (auto &op : plan.task(tg.task_id).ops) {
                        const bool comm = comm_ops.count(op.type) > 0;
                        auto touch = [&](const TensorDesc &t, bool is_write) {
                            Life &l = life[t.buffer_id];
                            if (comm || !whole(t)) l.ok = false;
                            if (l.first < 0) { l.first = step; l.first_is_write = is_write; }
                            l.last = step;
                            (is_write ? l.written : l.read) = true;
                        };
                        // reads first: an op that reads and writes one buffer (in place) needs the old contents
                        if (!op.is_virtual) {
                            for (auto &t : op.reads) touch(t, false);
                            for (auto &t : op.writes) touch(t, true);
                            for (auto &t : op.results) touch(t, true);
                        } else {
                            for (auto &t : op.reads) life[t.buffer_id].ok = life[t.buffer_id].ok && whole(t);
                            for (auto &t : op.results) life[t.buffer_id].ok = life[t.buffer_id].ok && whole(t);
                        }
                    }
            ++step;
        }
        // ops the schedule never runs (task infos without a task group) still pin their buffers
        std::set<int64_t> scheduled;
        for (auto &pg : plan.processor_groups)
            for (auto &rg : pg.resource_groups)
                for (auto &tg : rg.task_groups) scheduled.insert(tg.task_id);
        for (auto &ti : plan.task_infos)
            if (!scheduled.count(ti.id))
                for (auto &op : ti.ops) {
                    for (auto &t : op.reads) life[t.buffer_id].ok = false;
                    for (auto &t : op.writes) life[t.buffer_id].ok = false;
                    for (auto &t : op.results) life[t.buffer_id].ok = false;
                }
    }
    auto reusable = [&](const BufferInfo &b) {
        auto it = life.find(b.id);
        if (it == life.end()) return false;
        const Life &l = it->second;
        return plan.arena_reuse && l.ok && l.written && l.read && l.first_is_write && l.first >= 0 && b.send_tags.empty() &&
               b.recv_tags.empty() && (b.rank == -1 || b.rank == plan.rank);
    };
    size_t off = 0, off_plain = 0;
    std::vector<BufferInfo *> pool;
    for (auto &kv : lay.buffers) {  // std::map: buffer-id order, as the reference
        BufferInfo &b = kv.second;
        if (b.rank != -1 && b.rank != plan.rank) continue;  // remote: resolved later
        off_plain = align_up(off_plain + b.bytes, kArenaAlign);
        if (reusable(b)) {
            pool.push_back(&b);
            continue;
        }
        b.offset = off;
        b.resolved = true;
        off = align_up(off + b.bytes, kArenaAlign);
        for (auto &tg : b.send_tags) lay.published.push_back({0, tg.first, tg.second, 0, b.offset});
        for (auto &tg : b.recv_tags) lay.published.push_back({1, tg.first, tg.second, 0, b.offset});
    }
    lay.arena_bytes_no_reuse = off_plain;
    if (!pool.empty()) {
        // Intermediates in order of birth; a buffer takes the lowest-addressed hole of the shared region that is free
        // over its whole lifetime (holes are what buffers that died earlier left), else the region grows.
        std::sort(pool.begin(), pool.end(), [&](BufferInfo *a, BufferInfo *b) {
            const Life &la = life[a->id], &lb = life[b->id];
            return la.first != lb.first ? la.first < lb.first : a->bytes > b->bytes;
        });
        struct Placed { size_t off, size; int first, last; };
        std::vector<Placed> placed;
        const size_t base = off;
        size_t top = 0;
        for (BufferInfo *b : pool) {
            const Life &l = life[b->id];
            const size_t size = align_up(std::max<size_t>(b->bytes, 1), kArenaAlign);
            // blocks alive at any step of [first, last], sorted by offset
            std::vector<std::pair<size_t, size_t>> busy;
            for (auto &p : placed)
                // one step of slack on either side: stages of neighbouring processor groups may run side by side when
                // no data dependency orders them, and sharing memory between them would create one
                if (!(p.last + 1 < l.first || p.first > l.last + 1)) busy.push_back({p.off, p.off + p.size});
            std::sort(busy.begin(), busy.end());
            size_t at = 0;
            for (auto &iv : busy) {
                if (at + size <= iv.first) break;
                at = std::max(at, iv.second);
            }
            placed.push_back({at, size, l.first, l.last});
            top = std::max(top, at + size);
            b->offset = base + at;
            b->resolved = true;
            ++lay.reused_buffers;
        }
        off = align_up(base + top, kArenaAlign);
    }
    // collective tags: AllReduce publishes where its tensor lives
    for (auto &ti : plan.task_infos)
        for (auto &op : ti.ops)
            if (op.type == "AllReduce") {
                const TensorDesc &t = op.results.at(0);
                int64_t es[4], org;
                t.elem_strides(es, org);
                const BufferInfo &b = lay.buffers.at(t.buffer_id);
                lay.published.push_back({2, -1, (int)op.arg_int("Tag"), 0, b.offset + (uint64_t)org * dtype_size(t.dtype)});
            }
    // staging slots of fused Matmul + AllReduce pairs: one slot per rank, together the size of the tensor
    for (auto &ti : plan.task_infos)
        for (size_t i = 0; i < ti.ops.size(); ++i)
            if (fused_allreduce(plan, ti, i)) {
                const TensorDesc &t = ti.ops[i].results[0];
                off = align_up(off, 1024);
                lay.published.push_back({3, -1, (int)ti.ops[i + 1].arg_int("Tag"), 0, off});
                off = align_up(off + (size_t)t.nelems() * dtype_size(t.dtype), kArenaAlign);
            }
    lay.arena_bytes = std::max<size_t>(off, kArenaAlign);
    // one-shot staging: kMaxPeers slots of the largest small all_reduce, capped
    const size_t kOneShotMax = 512 * 1024;
    lay.comm_stage_bytes = align_up(std::min(oneshot_max, kOneShotMax), 256) * kMaxPeers;
    return lay;
}

void resolve_remote(const Plan &plan, Layout &lay, const std::vector<std::vector<TagRecord>> &records) {
    for (auto &kv : lay.buffers) {
        BufferInfo &b = kv.second;
        if (b.resolved) continue;
        const int r = b.rank;
        if (r < 0 || r >= (int)records.size()) throw Error(E_PLAN, "buffer on unknown rank " + std::to_string(r));
        // A local stand-in for a remote buffer carries the same tag the owner
        // published: recv tag (owner receives our send) or send tag (owner sends to us).
        bool found = false;
        for (auto &tg : b.recv_tags) {
            for (auto &rec : records[r])
                if (rec.kind == 1 && rec.tag == tg.second && (rec.peer == plan.rank || rec.peer == -1)) {
                    b.offset = rec.offset;
                    found = true;
                }
        }
        for (auto &tg : b.send_tags) {
            for (auto &rec : records[r])
                if (rec.kind == 0 && rec.tag == tg.second && (rec.peer == plan.rank || rec.peer == -1)) {
                    b.offset = rec.offset;
                    found = true;
                }
        }
        // A stand-in no record matches stays without an address, as in the reference (ark/api/executor.cpp:376-392,
        // 468-500: only tags a peer sent fill in offsets). Plans hold such buffers on purpose: the source tensor of a
        // RecvPacket, or of a Recv with Wait=false, only names the sender. Using one as an operand is an error then.
        b.resolved = found;
    }
    for (size_t r = 0; r < records.size(); ++r)
        for (auto &rec : records[r])
            if (rec.kind == 2 || rec.kind == 3) {
                auto &v = rec.kind == 2 ? lay.coll_offsets[rec.tag] : lay.coll_stage_offsets[rec.tag];
                v.resize(records.size(), 0);
                v[r] = rec.offset;
            }
}

}  // namespace arkb
