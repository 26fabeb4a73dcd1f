#include "controller.h"

#include <algorithm>
#include <sstream>
#include <unordered_set>

#include "logging.h"

namespace hvd {

namespace {

bool IsReduction(Response::Type t) {
  return t == Response::ALLREDUCE || t == Response::ADASUM;
}

bool Cacheable(Response::Type t) {
  return t == Response::ALLREDUCE || t == Response::ADASUM ||
         t == Response::ALLGATHER || t == Response::ALLTOALL ||
         t == Response::REDUCESCATTER;
}

std::string ShapeString(const std::vector<int64_t>& s) {
  return TensorShape(s).DebugString();
}

}  // namespace

int64_t Controller::TensorFusionThresholdBytes() const {
  int64_t proposed = params_.TensorFusionThresholdBytes();
  int64_t unit = static_cast<int64_t>(std::max(1, opts_.local_size)) *
                 FUSION_ATOMIC_UNIT;
  return RoundUp(proposed, unit);
}

void Controller::SynchronizeParameters() {
  ParameterManager::Params p;
  if (is_coordinator()) p = params_.GetParams();
  comm_->Bcast(&p, sizeof(p), 0);
  if (!is_coordinator()) params_.SetParams(p);
}

void Controller::CoordinateCacheAndState(CacheCoordinator& cc) {
  cc.sync([this](uint64_t* w, size_t n, bool is_and) {
    comm_->AllreduceBits(w, n, is_and);
  });
  // Entries any rank found stale are dropped everywhere; their requests go
  // back through the coordinator this cycle.
  for (auto bit : cc.invalid_bits()) cache_.erase_response(bit);
}

ResponseList Controller::ComputeResponseList(bool shutdown_requested,
                                             JoinState& join) {
  if (params_.IsAutoTuning())
    cache_.set_capacity(params_.CacheEnabled() ? opts_.cache_capacity : 0);
  const bool cache_on = cache_.capacity() > 0;

  CacheCoordinator cc(cache_.num_active_bits());
  std::deque<Request> msgs;
  queue_.PopMessagesFromQueue(msgs);

  for (auto& m : msgs) {
    if (m.type == Request::JOIN) {
      join.joined = true;
      cc.set_uncached_in_queue(true);
      continue;
    }
    if (!cache_on) continue;
    auto state = cache_.cached(m);
    if (state == ResponseCache::CacheState::HIT) {
      cc.record_hit(cache_.peek_cache_bit(m.name));
      stall_.RecordCachedTensorStart(m.name);
    } else {
      if (state == ResponseCache::CacheState::INVALID)
        cc.record_invalid_bit(cache_.peek_cache_bit(m.name));
      cc.set_uncached_in_queue(true);
      stall_.RemoveCachedTensor(m.name);
    }
  }
  // A rank that joined agrees to whatever cached reduction the others run (it
  // contributes zeros). Collectives that cannot run with a joined rank
  // (allgather, broadcast, alltoall, reducescatter) must not take the cache
  // fast path either: their cached responses are invalidated on every rank,
  // so that the next request for them goes through the coordinator and gets
  // the same error as an uncached one.
  if (join.joined && cache_on) {
    for (auto bit : cache_.list_all_bits()) {
      const Response::Type t = cache_.peek_response(bit).type;
      if (t == Response::ALLREDUCE || t == Response::ADASUM) {
        cc.record_hit(bit);
      } else {
        cc.record_invalid_bit(bit);
        cc.set_uncached_in_queue(true);
      }
    }
  }

  bool should_shut_down = shutdown_requested;
  if (stall_.ShouldPerformCheck()) {
    if (is_coordinator())
      should_shut_down |= stall_.CheckForStalledTensors(comm_->global_ranks());
    if (cache_on) stall_.InvalidateStalledCachedTensors(cc);
    stall_.UpdateCheckTime();
  }
  cc.set_should_shut_down(should_shut_down);

  if (cache_on) {
    CoordinateCacheAndState(cc);
    std::deque<Request> retry, uncached;
    for (auto& m : msgs) {
      bool hit = m.type != Request::JOIN &&
                 cache_.cached(m) == ResponseCache::CacheState::HIT;
      if (hit) {
        uint32_t bit = cache_.peek_cache_bit(m.name);
        if (cc.cache_hits().count(bit)) {
          stall_.RemoveCachedTensor(m.name);  // runs this cycle
        } else {
          retry.push_back(std::move(m));  // others are not ready yet
        }
      } else {
        stall_.RemoveCachedTensor(m.name);
        uncached.push_back(std::move(m));
      }
    }
    queue_.PushMessagesToQueue(retry);
    msgs.swap(uncached);
  }

  ResponseList result;
  result.shutdown = cc.should_shut_down() || (!cache_on && should_shut_down);

  const bool need_communication = !(cache_on && !cc.uncached_in_queue());
  if (!msgs.empty() || !cc.cache_hits().empty())
    HVD_LOG_RANK(TRACE, comm_->global_ranks()[comm_->rank()])
        << "negotiate: " << msgs.size() << " uncached request(s), "
        << cc.cache_hits().size() << " common cache hit(s), "
        << cache_.num_active_bits() << " cache bit(s), "
        << (need_communication ? "coordinator round" : "cache fast path")
        << (join.joined ? ", joined" : "");

  if (!need_communication) {
    if (cc.cache_hits().empty()) return result;
    // Fast path: every rank holds identical cached responses.
    if (opts_.disable_group_fusion && !groups_.empty()) {
      std::vector<int32_t> ready_groups;
      std::unordered_set<int32_t> seen;
      for (auto bit : cc.cache_hits()) {
        int32_t gid =
            groups_.GetGroupIDFromTensorName(cache_.peek_response(bit).names[0]);
        if (gid != NULL_GROUP_ID && seen.insert(gid).second)
          ready_groups.push_back(gid);
      }
      for (auto gid : ready_groups) {
        std::deque<Response> group;
        // A group is fused on its own only when every member is a common hit.
        // If one is not (evicted from the cache, say), the members that are
        // run below like ungrouped tensors: every rank holds the same cache
        // and the same hit set, so all ranks take the same decision.
        bool whole = true;
        for (auto& name : groups_.GetGroupTensorNames(gid))
          if (!cache_.has_name(name) || !cc.cache_hits().count(cache_.peek_cache_bit(name)))
            whole = false;
        if (!whole) continue;
        for (auto& name : groups_.GetGroupTensorNames(gid)) {
          uint32_t bit = cache_.peek_cache_bit(name);
          group.push_back(cache_.get_response(bit));
          cc.erase_hit(bit);
        }
        FuseResponses(group, result);
      }
    }
    std::deque<Response> responses;
    for (auto bit : cc.cache_hits())
      responses.push_back(cache_.get_response(bit));
    FuseResponses(responses, result);
    cache_.update_cache_bits();
    return result;
  }

  // Slow path: the coordinator decides.
  if (is_coordinator()) {
    std::vector<std::string> ready;
    auto absorb = [&](const Request& m, int from_rank) {
      if (m.type == Request::JOIN) {
        ++join.joined_size;
        join.last_joined_rank = from_rank;
        return;
      }
      bool complete = IncrementTensorCount(m, join.joined_size);
      stall_.RecordUncachedTensorStart(m.name, m.request_rank, size());
      if (complete) ready.push_back(m.name);
    };
    for (auto& m : msgs) absorb(m, 0);
    msgs.clear();

    std::vector<std::string> blobs;
    comm_->GatherBlobs(std::string(), 0, &blobs);
    for (int r = 1; r < size(); ++r) {
      RequestList rl = RequestList::Parse(blobs[r].data(), blobs[r].size());
      for (auto& m : rl.requests) absorb(m, r);
      if (rl.shutdown) should_shut_down = true;
    }

    // Tensors that were waiting only for ranks that have since joined.
    if (join.joined_size > 0) {
      for (auto& kv : message_table_) {
        if (static_cast<int>(kv.second.size()) == size() - join.joined_size &&
            std::find(ready.begin(), ready.end(), kv.first) == ready.end()) {
          timeline_.NegotiateEnd(kv.first);
          ready.push_back(kv.first);
        }
      }
    }

    if (opts_.disable_group_fusion && !groups_.empty()) {
      std::vector<int32_t> ready_groups;
      std::unordered_set<int32_t> seen;
      for (auto& name : ready) {
        int32_t gid = groups_.GetGroupIDFromTensorName(name);
        if (gid != NULL_GROUP_ID && seen.insert(gid).second)
          ready_groups.push_back(gid);
      }
      if (cache_on) {
        for (auto bit : cc.cache_hits()) {
          int32_t gid = groups_.GetGroupIDFromTensorName(
              cache_.peek_response(bit).names[0]);
          if (gid != NULL_GROUP_ID && seen.insert(gid).second)
            ready_groups.push_back(gid);
        }
      }
      for (auto gid : ready_groups) {
        std::deque<Response> group;
        for (auto& name : groups_.GetGroupTensorNames(gid)) {
          if (message_table_.count(name)) {
            group.push_back(ConstructResponse(name, join.joined_size));
          } else if (cache_on && cache_.has_name(name)) {
            uint32_t bit = cache_.peek_cache_bit(name);
            group.push_back(cache_.peek_response(bit));
            cc.erase_hit(bit);
          }
        }
        FuseResponses(group, result);
      }
    }

    std::deque<Response> responses;
    // Cached responses every rank is ready for ride along (peek, not get:
    // the cache order is refreshed by the put() all ranks do below).
    if (cache_on && join.joined_size < size())
      for (auto bit : cc.cache_hits())
        responses.push_back(cache_.peek_response(bit));

    for (auto& name : ready) {
      if (opts_.disable_group_fusion && !groups_.empty() &&
          groups_.GetGroupIDFromTensorName(name) != NULL_GROUP_ID)
        continue;  // went out with its group above
      if (!message_table_.count(name)) continue;
      responses.push_back(ConstructResponse(name, join.joined_size));
    }
    if (join.joined_size == size()) {
      Response jr;
      jr.type = Response::JOIN;
      jr.names.push_back(JOIN_TENSOR_NAME);
      jr.last_joined_rank = join.last_joined_rank;
      responses.push_back(std::move(jr));
      join.joined_size = 0;
    }
    FuseResponses(responses, result);
    result.shutdown = should_shut_down || cc.should_shut_down();

    std::string blob = result.Serialize();
    comm_->BcastBlob(&blob, 0);
  } else {
    RequestList rl;
    rl.shutdown = should_shut_down;
    for (auto& m : msgs) rl.requests.push_back(std::move(m));
    msgs.clear();
    std::vector<std::string> unused;
    comm_->GatherBlobs(rl.Serialize(), 0, &unused);
    std::string blob;
    comm_->BcastBlob(&blob, 0);
    result = ResponseList::Parse(blob.data(), blob.size());
  }

  if (cache_on) {
    // Same insertions in the same order on every rank keep bits aligned.
    for (auto& r : result.responses) {
      if (Cacheable(r.type) && static_cast<int>(r.devices.size()) == size())
        cache_.put(r, queue_, join.joined);
    }
  }
  cache_.update_cache_bits();
  return result;
}

bool Controller::IncrementTensorCount(const Request& msg, int joined_size) {
  auto it = message_table_.find(msg.name);
  if (it == message_table_.end()) {
    timeline_.NegotiateStart(msg.name, msg.type);
    it = message_table_.emplace(msg.name, std::vector<Request>()).first;
  }
  timeline_.NegotiateRankReady(msg.name, msg.request_rank);
  it->second.push_back(msg);
  bool complete =
      static_cast<int>(it->second.size()) == size() - joined_size;
  if (complete) timeline_.NegotiateEnd(msg.name);
  return complete;
}

Response Controller::ConstructResponse(const std::string& name,
                                       int joined_size) {
  auto node = message_table_.find(name);
  std::vector<Request> reqs = std::move(node->second);
  message_table_.erase(node);
  stall_.RemoveUncachedTensor(name);
  std::sort(reqs.begin(), reqs.end(), [](const Request& a, const Request& b) {
    return a.request_rank < b.request_rank;
  });

  const Request& first = reqs[0];
  std::ostringstream err;
  bool bad = false;

  for (size_t i = 1; i < reqs.size() && !bad; ++i) {
    if (reqs[i].dtype != first.dtype) {
      bad = true;
      err << "Mismatched data types: One rank had type "
          << DataTypeName(first.dtype) << ", but another rank had type "
          << DataTypeName(reqs[i].dtype) << ".";
    }
  }
  for (size_t i = 1; i < reqs.size() && !bad; ++i) {
    if (reqs[i].type != first.type) {
      bad = true;
      err << "Mismatched operations: One rank did an "
          << Request::TypeName(first.type) << ", but another rank did an "
          << Request::TypeName(reqs[i].type) << ".";
    }
  }

  const Request::Type type = first.type;
  const bool same_shape_needed =
      type == Request::ALLREDUCE || type == Request::ADASUM ||
      type == Request::BROADCAST || type == Request::REDUCESCATTER;
  if (!bad && same_shape_needed) {
    for (size_t i = 1; i < reqs.size() && !bad; ++i) {
      if (reqs[i].shape != first.shape) {
        bad = true;
        err << "Mismatched " << Request::TypeName(type)
            << " tensor shapes: One rank sent a tensor of shape "
            << ShapeString(first.shape)
            << ", but another rank sent a tensor of shape "
            << ShapeString(reqs[i].shape) << ".";
      }
    }
  }
  if (!bad && (type == Request::ALLREDUCE || type == Request::ADASUM ||
               type == Request::REDUCESCATTER)) {
    for (size_t i = 1; i < reqs.size() && !bad; ++i) {
      if (reqs[i].prescale != first.prescale ||
          reqs[i].postscale != first.postscale) {
        bad = true;
        err << "Mismatched prescale and/or postscale factors: One rank sent "
               "factors ("
            << first.prescale << ", " << first.postscale
            << "), but another rank sent factors (" << reqs[i].prescale
            << ", " << reqs[i].postscale << ").";
      } else if (reqs[i].wire_dtype != first.wire_dtype) {
        bad = true;
        err << "Mismatched compression: One rank sends "
            << DataTypeName(first.wire_dtype) << " on the wire, but another rank sends "
            << DataTypeName(reqs[i].wire_dtype) << ".";
      } else if (reqs[i].reduce_op != first.reduce_op) {
        bad = true;
        err << "Mismatched reduction operations: One rank requested "
            << ReduceOpName(first.reduce_op) << ", but another rank requested "
            << ReduceOpName(reqs[i].reduce_op) << ".";
      }
    }
  }

  std::vector<int64_t> tensor_sizes;
  if (!bad && (type == Request::ALLGATHER || type == Request::ALLTOALL ||
               type == Request::REDUCESCATTER)) {
    if (joined_size > 0) {
      bad = true;
      if (type == Request::ALLGATHER)
        err << "Allgather is not supported with Join at this time. Specify "
               "sparse_to_dense=True if using DistributedOptimizer";
      else if (type == Request::ALLTOALL)
        err << "Alltoall is not supported with Join at this time.";
      else
        err << "Reducescatter is not supported with Join at this time.";
    }
  }
  if (!bad && (type == Request::ALLGATHER || type == Request::ALLTOALL)) {
    if (first.shape.empty()) {
      bad = true;
      err << "Process-set rank zero tried to "
          << (type == Request::ALLGATHER ? "allgather" : "alltoall")
          << " a rank-zero tensor.";
    }
    for (size_t i = 1; i < reqs.size() && !bad; ++i) {
      if (reqs[i].shape.size() != first.shape.size()) {
        bad = true;
        err << "Mismatched " << Request::TypeName(type)
            << " tensor shapes: One rank sent a tensor of rank "
            << first.shape.size() << ", but another rank sent a tensor of rank "
            << reqs[i].shape.size() << ".";
        break;
      }
      for (size_t d = 1; d < first.shape.size(); ++d) {
        if (reqs[i].shape[d] != first.shape[d]) {
          bad = true;
          err << "Mismatched " << Request::TypeName(type)
              << " tensor shapes: One rank sent a tensor with dimension " << d
              << " equal to " << first.shape[d]
              << ", but another rank sent a tensor with dimension " << d
              << " equal to " << reqs[i].shape[d] << ".";
          break;
        }
      }
    }
    // First dimension of every rank's tensor, in rank order (for an alltoall:
    // what even splits are derived from).
    if (!bad)
      for (auto& q : reqs) tensor_sizes.push_back(q.shape[0]);
  }
  if (!bad && (type == Request::ALLREDUCE || type == Request::ADASUM ||
               type == Request::REDUCESCATTER)) {
    int64_t n = 1;
    for (auto d : first.shape) n *= d;
    tensor_sizes.push_back(n);
  }
  if (!bad && type == Request::REDUCESCATTER && first.shape.empty()) {
    bad = true;
    err << "Process-set rank zero tried to reducescatter a rank-zero tensor.";
  }
  if (!bad && type == Request::BROADCAST) {
    if (joined_size > 0) {
      bad = true;
      err << "Broadcast is not supported with Join at this time.";
    }
    for (size_t i = 1; i < reqs.size() && !bad; ++i) {
      if (reqs[i].root_rank != first.root_rank) {
        bad = true;
        err << "Mismatched " << Request::TypeName(type)
            << " root ranks: One rank specified root rank " << first.root_rank
            << ", but another rank specified root rank " << reqs[i].root_rank
            << ".";
      }
    }
    if (!bad) {
      int64_t n = 1;
      for (auto d : first.shape) n *= d;
      tensor_sizes.push_back(n * static_cast<int64_t>(DataTypeSize(first.dtype)));
    }
  }
  for (size_t i = 1; i < reqs.size() && !bad; ++i) {
    bool a = first.device == CPU_DEVICE_ID, b = reqs[i].device == CPU_DEVICE_ID;
    if (a != b) {
      bad = true;
      err << "Mismatched CPU/GPU device selection: One rank specified device "
          << (a ? "CPU" : "GPU") << ", but another rank specified device "
          << (b ? "CPU" : "GPU") << ".";
    }
  }

  Response resp;
  resp.names.push_back(name);
  if (bad) {
    resp.type = Response::ERROR;
    resp.error_message = err.str();
    return resp;
  }
  for (auto& q : reqs) resp.devices.push_back(q.device);
  resp.dtype = first.dtype;
  resp.tensor_sizes = std::move(tensor_sizes);
  resp.prescale = first.prescale;
  resp.postscale = first.postscale;
  resp.reduce_op = first.reduce_op;
  resp.root_rank = first.root_rank;
  if (type == Request::ALLTOALL) {
    // 1 only when every rank asked for an even split.
    resp.root_rank = 1;
    for (auto& q : reqs)
      if (q.root_rank != 1) resp.root_rank = 0;
  }
  resp.wire_dtype = (type == Request::ALLREDUCE) ? first.wire_dtype : first.dtype;
  switch (type) {
  case Request::ALLREDUCE: resp.type = Response::ALLREDUCE; break;
  case Request::ALLGATHER: resp.type = Response::ALLGATHER; break;
  case Request::BROADCAST: resp.type = Response::BROADCAST; break;
  case Request::ADASUM: resp.type = Response::ADASUM; break;
  case Request::ALLTOALL: resp.type = Response::ALLTOALL; break;
  case Request::REDUCESCATTER: resp.type = Response::REDUCESCATTER; break;
  case Request::JOIN: resp.type = Response::JOIN; break;
  }
  return resp;
}

int64_t Controller::ResponseBytes(const Response& r) const {
  int64_t es = static_cast<int64_t>(DataTypeSize(r.dtype));
  int64_t total = 0;
  if (IsReduction(r.type) || r.type == Response::REDUCESCATTER) {
    int64_t ws = r.type == Response::ALLREDUCE
                     ? static_cast<int64_t>(DataTypeSize(r.wire_dtype)) : es;
    for (auto n : r.tensor_sizes) total += RoundUp(n * ws, FUSION_ALIGN_BYTES);
  } else if (r.type == Response::BROADCAST) {
    for (auto n : r.tensor_sizes) total += RoundUp(n, FUSION_ALIGN_BYTES);
  } else if (r.type == Response::ALLGATHER) {
    // Output bytes: sum over ranks of dim0 times the slice size, which only
    // the pending entry knows.
    size_t per = r.names.empty() ? 0 : r.tensor_sizes.size() / r.names.size();
    for (size_t i = 0; i < r.names.size(); ++i) {
      int64_t slice = 1;
      if (queue_.IsTensorPresentInTable(r.names[i])) {
        TensorTableEntry meta = queue_.GetTensorEntry(r.names[i]);
        for (int d = 1; d < meta.shape.dims(); ++d) slice *= meta.shape.dim_size(d);
      }
      int64_t rows = 0;
      for (size_t k = 0; k < per; ++k) rows += r.tensor_sizes[i * per + k];
      total += rows * slice * es;
    }
  }
  return total;
}

void Controller::FuseResponses(std::deque<Response>& responses,
                               ResponseList& out) {
  FuseResponseQueue(responses, TensorFusionThresholdBytes(),
                    [this](const Response& r) { return ResponseBytes(r); }, out);
}

void FuseResponseQueue(std::deque<Response>& responses, int64_t threshold,
                       const std::function<int64_t(const Response&)>& ResponseBytes,
                       ResponseList& out) {
  while (!responses.empty()) {
    Response r = std::move(responses.front());
    responses.pop_front();
    // Reduce-scatters fuse like allreduces (same dtype, scaling and op): the
    // ops take a fused response as a list of tensors to shard one by one, or,
    // on a device, in one launch.
    const bool reduction = IsReduction(r.type) || r.type == Response::REDUCESCATTER;
    const bool fusable = reduction || r.type == Response::ALLGATHER ||
                         r.type == Response::BROADCAST;
    if (fusable) {
      int64_t bytes = ResponseBytes(r);
      int64_t skipped_bytes = 0;
      std::deque<Response> skipped;
      while (!responses.empty()) {
        Response& next = responses.front();
        int64_t nb = ResponseBytes(next);
        bool compatible = next.type == r.type && next.devices == r.devices;
        if (compatible && r.type != Response::BROADCAST)
          compatible = next.dtype == r.dtype;
        if (compatible && reduction)
          compatible = next.prescale == r.prescale &&
                       next.postscale == r.postscale &&
                       next.reduce_op == r.reduce_op &&
                       next.wire_dtype == r.wire_dtype;
        if (compatible && r.type == Response::BROADCAST)
          compatible = next.root_rank == r.root_rank;
        if (compatible && bytes + nb <= threshold) {
          bytes += nb;
          for (auto& n : next.names) r.names.push_back(std::move(n));
          for (auto s : next.tensor_sizes) r.tensor_sizes.push_back(s);
          responses.pop_front();
        } else {
          // Look past a response that does not fit (mixed dtypes interleave
          // in mixed-precision training) as long as what was skipped would
          // still have fitted.
          skipped_bytes += nb;
          if (bytes + skipped_bytes <= threshold) {
            skipped.push_back(std::move(next));
            responses.pop_front();
          } else {
            break;
          }
        }
      }
      while (!skipped.empty()) {
        responses.push_front(std::move(skipped.back()));
        skipped.pop_back();
      }
    }
    out.responses.push_back(std::move(r));
  }
}

}  // namespace hvd
