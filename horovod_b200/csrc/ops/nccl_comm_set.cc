#include "nccl_comm_set.h"

#include <string>

#include "../common/logging.h"
#include "nccl_api.h"

namespace hvd {

void* NcclCommSet::Find(int32_t key) {
  std::lock_guard<std::mutex> l(mu_);
  auto it = comms_.find(key);
  return it == comms_.end() ? nullptr : it->second;
}

void NcclCommSet::Put(int32_t key, void* comm) {
  std::lock_guard<std::mutex> l(mu_);
  comms_[key] = comm;
}

bool NcclCommSet::empty() {
  std::lock_guard<std::mutex> l(mu_);
  return comms_.empty();
}

bool NcclCommSet::failed() {
  std::lock_guard<std::mutex> l(mu_);
  return failed_;
}

Status NcclCommSet::CheckAsyncErrors() {
  if (api_ == nullptr || api_->CommGetAsyncError == nullptr) return Status::OK();
  std::string what;
  {
    std::lock_guard<std::mutex> l(mu_);
    for (auto& kv : comms_) {
      ncclResult_t async = ncclSuccess;
      ncclResult_t rc = api_->CommGetAsyncError(static_cast<ncclComm_t>(kv.second), &async);
      if (rc != ncclSuccess) async = rc;
      if (async != ncclSuccess && async != ncclInProgress) {
        what = api_->GetErrorString ? api_->GetErrorString(async) : "unknown";
        break;
      }
    }
  }
  if (what.empty()) return Status::OK();
  {
    // Wait for a response that is being issued right now, then tear down.
    std::lock_guard<std::mutex> issue(issue_mu_);
    std::lock_guard<std::mutex> l(mu_);
    for (auto& kv : comms_)
      if (kv.second && api_->CommAbort) api_->CommAbort(static_cast<ncclComm_t>(kv.second));
    comms_.clear();
    failed_ = true;
  }
  HVD_LOG(ERROR) << "NCCL reported an asynchronous error (" << what
                 << "); its communicators were aborted.";
  return Status::UnknownError("NCCL reported an asynchronous error (" + what +
                              "); the communicators were aborted.");
}

void NcclCommSet::DestroyAll() {
  std::lock_guard<std::mutex> l(mu_);
  if (api_ != nullptr && api_->CommDestroy != nullptr)
    for (auto& kv : comms_)
      if (kv.second) api_->CommDestroy(static_cast<ncclComm_t>(kv.second));
  comms_.clear();
  failed_ = false;
}

}  // namespace hvd
